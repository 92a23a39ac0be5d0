// extern "C" entry points of the memory-rule kernels (Delta / DGD, Titans LMM,
// Hebbian; exact, checkpointed, segment, frozen-M0 chunkwise, phase-2, fused).
// Signatures follow core/src/cuda_ffi.rs; see include/nlh_ffi.h.
//
// Dispatch: register-resident kernels (memory_fast.cuh) when the head
// dimension and options allow it, the generic-d kernels otherwise.
#include "memory_generic.cuh"
#include "memory_exact_bwd.cuh"
#include "chunk_mm.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {

struct WsCarver {
    char* base; size_t off;
    explicit WsCarver(void* p) : base((char*)p), off(0) {}
    float* take(size_t floats) {
        float* r = (float*)(base + off);
        off += (floats * sizeof(float) + 255) & ~(size_t)255;
        return r;
    }
    static size_t need(size_t floats) { return (floats * sizeof(float) + 255) & ~(size_t)255; }
};

static bool valid_dims(const char* where, int seq_len, int d, int batch)
{
    if (d <= 0 || seq_len < 0 || batch < 0) {
        record_status(NLH_ERR_INVALID_ARG, where, "d must be > 0, seq_len and batch_size >= 0");
        return false;
    }
    if (gen_bwd_smem(d) > 200 * 1024) {
        record_status(NLH_ERR_INVALID_ARG, where, "d too large for the shared-memory staging");
        return false;
    }
    return true;
}

template <int RULE>
static bool launch_gen_fwd(const FwdArgs& a, cudaStream_t st)
{
    const size_t smem = gen_fwd_smem(a.d);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(gen_fwd_kernel<RULE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    gen_fwd_kernel<RULE><<<a.batch, GEN_THREADS, smem, st>>>(a);
    return check_launch("gen_fwd_kernel");
}

template <int RULE>
static bool launch_gen_bwd(const BwdArgs& a, cudaStream_t st)
{
    const size_t smem = gen_bwd_smem(a.d);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(gen_bwd_kernel<RULE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    gen_bwd_kernel<RULE><<<a.batch, GEN_THREADS, smem, st>>>(a);
    return check_launch("gen_bwd_kernel");
}

// Forward of any rule/mode. Returns an NLH status.
static int run_forward(int rule, FwdArgs a, const char* where)
{
    if (!valid_dims(where, a.seq_len, a.d, a.batch)) return NLH_ERR_INVALID_ARG;
    if (a.batch == 0) return NLH_OK;
    if ((a.store_mode == STORE_CKPT || a.store_mode == STORE_CHUNK) && a.interval <= 0) {
        record_status(NLH_ERR_INVALID_ARG, where, "interval / chunk_size must be > 0");
        return NLH_ERR_INVALID_ARG;
    }
    cudaStream_t st = current_stream();
    if (option_value(NLH_OPT_CHUNK_MATRIX) && cmm::forward(rule, a, st))
        return check_launch(where) ? NLH_OK : NLH_ERR_CUDA;
    if (fast_forward(rule, a, st)) return check_launch(where) ? NLH_OK : NLH_ERR_CUDA;
    if (rule == RULE_TITANS && a.s_out == nullptr) {
        record_status(NLH_ERR_UNSUPPORTED, where,
                      "s_states == NULL needs the register-resident path (head_dim 32/64, no clip/projection, aligned)");
        return NLH_ERR_UNSUPPORTED;
    }
    const size_t dd = (size_t)a.d * a.d;
    if (a.store_mode != STORE_ALL) {
        const size_t per = WsCarver::need((size_t)a.batch * dd);
        void* ws = workspace(per * 2);
        if (!ws) return NLH_ERR_WORKSPACE;
        WsCarver c(ws);
        a.m_work = c.take((size_t)a.batch * dd);
        a.s_work = c.take((size_t)a.batch * dd);
    }
    bool ok = false;
    if (rule == RULE_TITANS) ok = launch_gen_fwd<RULE_TITANS>(a, st);
    else if (rule == RULE_DELTA) ok = launch_gen_fwd<RULE_DELTA>(a, st);
    else if (rule == RULE_HEBBIAN) ok = launch_gen_fwd<RULE_HEBBIAN>(a, st);
    else { record_status(NLH_ERR_INVALID_ARG, where, "unknown rule"); return NLH_ERR_INVALID_ARG; }
    return ok ? NLH_OK : NLH_ERR_CUDA;
}

static int run_backward(int rule, BwdArgs a, const char* where)
{
    if (!valid_dims(where, a.seq_len, a.d, a.batch)) return NLH_ERR_INVALID_ARG;
    if (a.batch == 0) return NLH_OK;
    if (a.frozen && a.chunk <= 0) {
        record_status(NLH_ERR_INVALID_ARG, where, "chunk_size must be > 0");
        return NLH_ERR_INVALID_ARG;
    }
    cudaStream_t st = current_stream();
    if (option_value(NLH_OPT_CHUNK_MATRIX) && cmm::backward(rule, a, st))
        return check_launch(where) ? NLH_OK : NLH_ERR_CUDA;
    if (fast_backward(rule, a, st)) return check_launch(where) ? NLH_OK : NLH_ERR_CUDA;
    if (rule == RULE_TITANS && a.s_traj == nullptr) {
        record_status(NLH_ERR_UNSUPPORTED, where,
                      "s_states == NULL needs the register-resident path (head_dim 32/64, no clip/projection, aligned)");
        return NLH_ERR_UNSUPPORTED;
    }
    const size_t dd = (size_t)a.d * a.d;
    const size_t nb = (size_t)a.batch * dd;
    size_t bytes = WsCarver::need(nb) * 3;
    if (a.chunk > 0) bytes += WsCarver::need(nb * (a.chunk + 1)) * 2;
    void* ws = workspace(bytes);
    if (!ws) return NLH_ERR_WORKSPACE;
    WsCarver c(ws);
    a.dM = c.take(nb); a.dS = c.take(nb); a.dM0 = c.take(nb);
    if (a.chunk > 0) { a.m_rec = c.take(nb * (a.chunk + 1)); a.s_rec = c.take(nb * (a.chunk + 1)); }
    bool ok = false;
    if (rule == RULE_TITANS) ok = launch_gen_bwd<RULE_TITANS>(a, st);
    else if (rule == RULE_DELTA) ok = launch_gen_bwd<RULE_DELTA>(a, st);
    else if (rule == RULE_HEBBIAN) ok = launch_gen_bwd<RULE_HEBBIAN>(a, st);
    else { record_status(NLH_ERR_INVALID_ARG, where, "unknown rule"); return NLH_ERR_INVALID_ARG; }
    return ok ? NLH_OK : NLH_ERR_CUDA;
}

static FwdArgs fwd_args(const float* k, const float* v, const float* q, const float* alpha,
                        const float* theta, const float* eta, const float* m0, const float* s0,
                        float* m_out, float* s_out, float* y, int seq_len, int d, int batch,
                        long long in_stride, long long init_stride, long long out_stride, int mode,
                        int interval, int frozen, float clip, float mmax)
{
    FwdArgs a;
    a.k = k; a.v = v; a.q = q; a.alpha = alpha; a.theta = theta; a.eta = eta;
    a.m_init = m0; a.s_init = s0; a.m_out = m_out; a.s_out = s_out; a.y = y;
    a.m_work = nullptr; a.s_work = nullptr;
    a.seq_len = seq_len; a.d = d; a.batch = batch;
    a.in_stride_tok = in_stride; a.init_stride = init_stride; a.out_stride = out_stride;
    a.store_mode = mode; a.interval = interval; a.frozen = frozen;
    a.error_clip = clip; a.m_norm_max = mmax;
    return a;
}

static BwdArgs bwd_args(const float* k, const float* v, const float* q, const float* alpha,
                        const float* theta, const float* eta, const float* m_traj,
                        const float* s_traj, const float* d_y, const float* d_m_seed,
                        const float* d_s_seed, float* d_k, float* d_v, float* d_q, float* d_alpha,
                        float* d_theta, float* d_eta, float* d_m_out, float* d_s_out, int seq_len,
                        int d, int batch, int t_start, int t_end, long long traj_stride, int frozen,
                        int chunk, int atomic_out, float clip, float mmax)
{
    BwdArgs a;
    a.k = k; a.v = v; a.q = q; a.alpha = alpha; a.theta = theta; a.eta = eta;
    a.m_traj = m_traj; a.s_traj = s_traj; a.d_y = d_y; a.d_m_seed = d_m_seed; a.d_s_seed = d_s_seed;
    a.d_k = d_k; a.d_v = d_v; a.d_q = d_q; a.d_alpha = d_alpha; a.d_theta = d_theta; a.d_eta = d_eta;
    a.d_m_out = d_m_out; a.d_s_out = d_s_out;
    a.dM = a.dS = a.dM0 = a.m_rec = a.s_rec = nullptr;
    a.seq_len = seq_len; a.d = d; a.batch = batch; a.t_start = t_start; a.t_end = t_end;
    a.traj_stride = traj_stride; a.frozen = frozen; a.chunk = chunk; a.atomic_out = atomic_out;
    a.error_clip = clip; a.m_norm_max = mmax;
    return a;
}

static long long ckpt_slots(int seq_len, int interval)
{
    return (long long)(seq_len + interval - 1) / interval + 1;
}

// ── fused-forward pre-step: L2-normalise k,q rows in place and compute the gates ──
// One warp per token. Gate activations follow core/src/tensor.rs:199-227
// (sigmoid / softplus saturating at |x| >= 15).
__device__ __forceinline__ float sigmoid_sat(float x)
{
    if (x >= 15.0f) return 1.0f;
    if (x <= -15.0f) return 0.0f;
    return 1.0f / (1.0f + expf(-x));
}
__device__ __forceinline__ float softplus_sat(float x)
{
    if (x >= 15.0f) return x;
    if (x <= -15.0f) return 0.0f;
    return logf(1.0f + expf(x));
}

__global__ void __launch_bounds__(256) fused_prep_kernel(
    float* k, const float* __restrict__ v, float* q,
    const float* __restrict__ w_alpha, const float* __restrict__ b_alpha,
    const float* __restrict__ w_theta, const float* __restrict__ b_theta,
    const float* __restrict__ w_eta, const float* __restrict__ b_eta,
    float a_lo, float a_hi, float t_lo, float t_hi,
    float* alpha_out, float* theta_out, float* eta_out, float* k_norms, float* q_norms,
    long long n_tok, int d)
{
    const int lane = threadIdx.x & 31;
    const long long tok = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (tok >= n_tok) return;
    float* kr = k + tok * d; float* qr = q + tok * d; const float* vr = v + tok * d;
    float ks = 0.0f, qs = 0.0f;
    for (int j = lane; j < d; j += 32) { ks += kr[j] * kr[j]; qs += qr[j] * qr[j]; }
    const float kn = sqrtf(warp_sum(ks)), qn = sqrtf(warp_sum(qs));
    const float ki = 1.0f / fmaxf(kn, 1e-8f), qi = 1.0f / fmaxf(qn, 1e-8f);
    float da = 0.0f, dt = 0.0f, de = 0.0f;
    for (int j = lane; j < d; j += 32) {
        const float kh = kr[j] * ki, vv = vr[j];
        kr[j] = kh;
        qr[j] = qr[j] * qi;
        da += kh * w_alpha[j] + vv * w_alpha[d + j];
        dt += kh * w_theta[j] + vv * w_theta[d + j];
        if (w_eta != nullptr) de += kh * w_eta[j] + vv * w_eta[d + j];
    }
    da = warp_sum(da); dt = warp_sum(dt);
    if (w_eta != nullptr) de = warp_sum(de);
    if (lane == 0) {
        k_norms[tok] = kn; q_norms[tok] = qn;
        alpha_out[tok] = fminf(fmaxf(sigmoid_sat(da + *b_alpha), a_lo), a_hi);
        theta_out[tok] = fminf(fmaxf(softplus_sat(dt + *b_theta), t_lo), t_hi);
        if (w_eta != nullptr) eta_out[tok] = sigmoid_sat(de + *b_eta);
    }
}

}  // namespace nlh

using namespace nlh;

extern "C" {

// ───────────────────────── exact, full trajectory ─────────────────────────
void delta_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int32_t seq_len, int32_t d, int32_t batch_size, int32_t input_stride, int32_t m_stride,
    float error_clip, float m_norm_max)
{
    run_forward(RULE_DELTA, fwd_args(k_mem, v_mem, q_mem, alpha, theta, nullptr, m_initial, nullptr,
        m_states, nullptr, y, seq_len, d, batch_size, input_stride, m_stride,
        (long long)(seq_len + 1) * d * d, STORE_ALL, 0, 0, error_clip, m_norm_max),
        "delta_forward_f32_cuda");
}

void dgd_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int32_t seq_len, int32_t d, int32_t batch_size, int32_t input_stride, int32_t m_stride,
    float error_clip)
{
    run_forward(RULE_DELTA, fwd_args(k_mem, v_mem, q_mem, alpha, theta, nullptr, m_initial, nullptr,
        m_states, nullptr, y, seq_len, d, batch_size, input_stride, m_stride,
        (long long)(seq_len + 1) * d * d, STORE_ALL, 0, 0, error_clip, 0.0f),
        "dgd_forward_f32_cuda");
}

void titans_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_states, float* s_states, float* y, int32_t seq_len, int32_t d,
    int32_t batch_size, int32_t input_stride, int32_t m_stride, float error_clip,
    float m_norm_max)
{
    run_forward(RULE_TITANS, fwd_args(k_mem, v_mem, q_mem, alpha, theta, eta, m_initial, s_initial,
        m_states, s_states, y, seq_len, d, batch_size, input_stride, m_stride,
        (long long)(seq_len + 1) * d * d, STORE_ALL, 0, 0, error_clip, m_norm_max),
        "titans_forward_f32_cuda");
}

void hebbian_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_initial, float* m_states, float* y, int32_t seq_len,
    int32_t d, int32_t batch_size, int32_t input_stride, int32_t m_stride)
{
    run_forward(RULE_HEBBIAN, fwd_args(k_mem, v_mem, q_mem, alpha, nullptr, nullptr, m_initial,
        nullptr, m_states, nullptr, y, seq_len, d, batch_size, input_stride, m_stride,
        (long long)(seq_len + 1) * d * d, STORE_ALL, 0, 0, 0.0f, 0.0f),
        "hebbian_forward_f32_cuda");
}

void delta_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta,
    float* d_m_initial, int32_t seq_len, int32_t d, int32_t batch_size, float error_clip)
{
    run_backward(RULE_DELTA, bwd_args(k_mem, v_mem, q_mem, alpha, theta, nullptr, m_states, nullptr,
        d_y, nullptr, nullptr, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, nullptr, d_m_initial,
        nullptr, seq_len, d, batch_size, 0, seq_len, (long long)(seq_len + 1) * d * d, 0, 0, 1,
        error_clip, 0.0f), "delta_backward_f32_cuda");
}

void dgd_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta,
    float* d_m_initial, int32_t seq_len, int32_t d, float error_clip)
{
    run_backward(RULE_DELTA, bwd_args(k_mem, v_mem, q_mem, alpha, theta, nullptr, m_states, nullptr,
        d_y, nullptr, nullptr, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, nullptr, d_m_initial,
        nullptr, seq_len, d, 1, 0, seq_len, (long long)(seq_len + 1) * d * d, 0, 0, 1,
        error_clip, 0.0f), "dgd_backward_f32_cuda");
}

void titans_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_states,
    const float* s_states, const float* d_y, float* d_k_mem, float* d_v_mem, float* d_q_mem,
    float* d_alpha, float* d_theta, float* d_eta, float* d_m_initial, float* d_s_initial,
    int32_t seq_len, int32_t d, int32_t batch_size, float error_clip)
{
    run_backward(RULE_TITANS, bwd_args(k_mem, v_mem, q_mem, alpha, theta, eta, m_states, s_states,
        d_y, nullptr, nullptr, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, d_eta, d_m_initial,
        d_s_initial, seq_len, d, batch_size, 0, seq_len, (long long)(seq_len + 1) * d * d, 0, 0, 1,
        error_clip, 0.0f), "titans_backward_f32_cuda");
}

void hebbian_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_states, const float* d_y, float* d_k_mem, float* d_v_mem,
    float* d_q_mem, float* d_alpha, float* d_m_initial, int32_t seq_len, int32_t d)
{
    run_backward(RULE_HEBBIAN, bwd_args(k_mem, v_mem, q_mem, alpha, nullptr, nullptr, m_states,
        nullptr, d_y, nullptr, nullptr, d_k_mem, d_v_mem, d_q_mem, d_alpha, nullptr, nullptr,
        d_m_initial, nullptr, seq_len, d, 1, 0, seq_len, (long long)(seq_len + 1) * d * d, 0, 0, 1,
        0.0f, 0.0f), "hebbian_backward_f32_cuda");
}

// ───────────────────────── checkpointed forward / segment backward ────────
void delta_forward_ckpt_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int32_t seq_len, int32_t d, int32_t checkpoint_interval, float error_clip, float m_norm_max)
{
    run_forward(RULE_DELTA, fwd_args(k_mem, v_mem, q_mem, alpha, theta, nullptr, m_initial, nullptr,
        m_states, nullptr, y, seq_len, d, 1, seq_len, (long long)d * d, 0, STORE_CKPT,
        checkpoint_interval, 0, error_clip, m_norm_max), "delta_forward_ckpt_f32_cuda");
}

void dgd_forward_ckpt_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int32_t seq_len, int32_t d, int32_t checkpoint_interval, float error_clip)
{
    run_forward(RULE_DELTA, fwd_args(k_mem, v_mem, q_mem, alpha, theta, nullptr, m_initial, nullptr,
        m_states, nullptr, y, seq_len, d, 1, seq_len, (long long)d * d, 0, STORE_CKPT,
        checkpoint_interval, 0, error_clip, 0.0f), "dgd_forward_ckpt_f32_cuda");
}

void titans_forward_ckpt_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_states, float* s_states, float* y, int32_t seq_len, int32_t d,
    int32_t checkpoint_interval, float error_clip, float m_norm_max)
{
    run_forward(RULE_TITANS, fwd_args(k_mem, v_mem, q_mem, alpha, theta, eta, m_initial, s_initial,
        m_states, s_states, y, seq_len, d, 1, seq_len, (long long)d * d, 0, STORE_CKPT,
        checkpoint_interval, 0, error_clip, m_norm_max), "titans_forward_ckpt_f32_cuda");
}

void hebbian_forward_ckpt_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_initial, float* m_states, float* y, int32_t seq_len,
    int32_t d, int32_t checkpoint_interval)
{
    run_forward(RULE_HEBBIAN, fwd_args(k_mem, v_mem, q_mem, alpha, nullptr, nullptr, m_initial,
        nullptr, m_states, nullptr, y, seq_len, d, 1, seq_len, (long long)d * d, 0, STORE_CKPT,
        checkpoint_interval, 0, 0.0f, 0.0f), "hebbian_forward_ckpt_f32_cuda");
}

void delta_backward_segment_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y,
    const float* d_m_seed, float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha,
    float* d_theta, float* d_m_out, int32_t t_start, int32_t t_end, int32_t d, int32_t batch_size,
    int32_t seq_len, float error_clip)
{
    run_backward(RULE_DELTA, bwd_args(k_mem, v_mem, q_mem, alpha, theta, nullptr, m_states, nullptr,
        d_y, d_m_seed, nullptr, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, nullptr, d_m_out,
        nullptr, seq_len, d, batch_size, t_start, t_end, (long long)(t_end - t_start + 1) * d * d,
        0, 0, 0, error_clip, 0.0f), "delta_backward_segment_f32_cuda");
}

void dgd_backward_segment_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y,
    const float* d_m_seed, float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha,
    float* d_theta, float* d_m_out, int32_t t_start, int32_t t_end, int32_t d, int32_t batch_size,
    int32_t seq_len, float error_clip)
{
    run_backward(RULE_DELTA, bwd_args(k_mem, v_mem, q_mem, alpha, theta, nullptr, m_states, nullptr,
        d_y, d_m_seed, nullptr, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, nullptr, d_m_out,
        nullptr, seq_len, d, batch_size, t_start, t_end, (long long)(t_end - t_start + 1) * d * d,
        0, 0, 0, error_clip, 0.0f), "dgd_backward_segment_f32_cuda");
}

void titans_backward_segment_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_states,
    const float* s_states, const float* d_y, const float* d_m_seed, const float* d_s_seed,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta,
    float* d_m_out, float* d_s_out, int32_t t_start, int32_t t_end, int32_t d, int32_t batch_size,
    int32_t seq_len, float error_clip)
{
    run_backward(RULE_TITANS, bwd_args(k_mem, v_mem, q_mem, alpha, theta, eta, m_states, s_states,
        d_y, d_m_seed, d_s_seed, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, d_eta, d_m_out,
        d_s_out, seq_len, d, batch_size, t_start, t_end,
        (long long)(t_end - t_start + 1) * d * d, 0, 0, 0, error_clip, 0.0f),
        "titans_backward_segment_f32_cuda");
}

void hebbian_backward_segment_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_states, const float* d_y, const float* d_m_seed,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_m_out,
    int32_t t_start, int32_t t_end, int32_t d, int32_t batch_size, int32_t seq_len)
{
    run_backward(RULE_HEBBIAN, bwd_args(k_mem, v_mem, q_mem, alpha, nullptr, nullptr, m_states,
        nullptr, d_y, d_m_seed, nullptr, d_k_mem, d_v_mem, d_q_mem, d_alpha, nullptr, nullptr,
        d_m_out, nullptr, seq_len, d, batch_size, t_start, t_end,
        (long long)(t_end - t_start + 1) * d * d, 0, 0, 0, 0.0f, 0.0f),
        "hebbian_backward_segment_f32_cuda");
}

// ───────────────────────── frozen-M0 chunkwise ────────────────────────────
void delta_chunkwise_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_chunk_states,
    float* y, int32_t seq_len, int32_t d, int32_t batch_size, int32_t chunk_size,
    float error_clip, float m_norm_max)
{
    if (chunk_size <= 0) { record_status(NLH_ERR_INVALID_ARG, "delta_chunkwise_forward_f32_cuda", "chunk_size must be > 0"); return; }
    run_forward(RULE_DELTA, fwd_args(k_mem, v_mem, q_mem, alpha, theta, nullptr, m_initial, nullptr,
        m_chunk_states, nullptr, y, seq_len, d, batch_size, seq_len, (long long)d * d,
        ckpt_slots(seq_len, chunk_size) * d * d, STORE_CHUNK, chunk_size, 1, error_clip,
        m_norm_max), "delta_chunkwise_forward_f32_cuda");
}

void titans_chunkwise_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_chunk_states, float* s_chunk_states, float* y,
    int32_t seq_len, int32_t d, int32_t batch_size, int32_t chunk_size, float error_clip,
    float m_norm_max)
{
    if (chunk_size <= 0) { record_status(NLH_ERR_INVALID_ARG, "titans_chunkwise_forward_f32_cuda", "chunk_size must be > 0"); return; }
    run_forward(RULE_TITANS, fwd_args(k_mem, v_mem, q_mem, alpha, theta, eta, m_initial, s_initial,
        m_chunk_states, s_chunk_states, y, seq_len, d, batch_size, seq_len, (long long)d * d,
        ckpt_slots(seq_len, chunk_size) * d * d, STORE_CHUNK, chunk_size, 1, error_clip,
        m_norm_max), "titans_chunkwise_forward_f32_cuda");
}

void delta_chunkwise_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_chunk_states, const float* d_y,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta,
    float* d_m_initial, int32_t seq_len, int32_t d, int32_t batch_size, int32_t chunk_size,
    float error_clip, float m_norm_max)
{
    if (chunk_size <= 0) { record_status(NLH_ERR_INVALID_ARG, "delta_chunkwise_backward_f32_cuda", "chunk_size must be > 0"); return; }
    run_backward(RULE_DELTA, bwd_args(k_mem, v_mem, q_mem, alpha, theta, nullptr, m_chunk_states,
        nullptr, d_y, nullptr, nullptr, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, nullptr,
        d_m_initial, nullptr, seq_len, d, batch_size, 0, seq_len,
        ckpt_slots(seq_len, chunk_size) * d * d, 1, chunk_size, 1, error_clip, m_norm_max),
        "delta_chunkwise_backward_f32_cuda");
}

void titans_chunkwise_backward_f32_cuda(const float* k_mem, const float* v_mem,
    const float* q_mem, const float* alpha, const float* theta, const float* eta,
    const float* m_chunk_states, const float* s_chunk_states, const float* d_y, float* d_k_mem,
    float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta,
    float* d_m_initial, float* d_s_initial, int32_t seq_len, int32_t d, int32_t batch_size,
    int32_t chunk_size, float error_clip, float m_norm_max)
{
    if (chunk_size <= 0) { record_status(NLH_ERR_INVALID_ARG, "titans_chunkwise_backward_f32_cuda", "chunk_size must be > 0"); return; }
    run_backward(RULE_TITANS, bwd_args(k_mem, v_mem, q_mem, alpha, theta, eta, m_chunk_states,
        s_chunk_states, d_y, nullptr, nullptr, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, d_eta,
        d_m_initial, d_s_initial, seq_len, d, batch_size, 0, seq_len,
        ckpt_slots(seq_len, chunk_size) * d * d, 1, chunk_size, 1, error_clip, m_norm_max),
        "titans_chunkwise_backward_f32_cuda");
}

// ───────────────────────── phase-1 epilogue, phase-2 per-chunk kernels ────
void error_subtract_clip_f32_cuda(float* predictions, const float* v, int32_t total_rows,
    int32_t d, float error_clip)
{
    if (total_rows <= 0 || d <= 0) return;
    const int wpb = 8;
    error_subtract_clip_kernel<<<(total_rows + wpb - 1) / wpb, wpb * 32, 0, current_stream()>>>(
        predictions, v, total_rows, d, error_clip);
    check_launch("error_subtract_clip_f32_cuda");
}

void delta_phase2_forward_f32_cuda(const float* k_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* errors, float* m_work, float* m_chunk_states, float* y,
    int32_t seq_len, int32_t d, int32_t batch_size, int32_t chunk_size, int32_t chunk_idx,
    float m_norm_max)
{
    if (!valid_dims("delta_phase2_forward_f32_cuda", seq_len, d, batch_size) || batch_size == 0) return;
    if (chunk_size <= 0 || chunk_idx < 0) { record_status(NLH_ERR_INVALID_ARG, "delta_phase2_forward_f32_cuda", "bad chunk"); return; }
    const size_t smem = gen_fwd_smem(d);
    if (smem > 48 * 1024) cudaFuncSetAttribute(gen_phase2_fwd_kernel<RULE_DELTA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gen_phase2_fwd_kernel<RULE_DELTA><<<batch_size, GEN_THREADS, smem, current_stream()>>>(
        k_mem, q_mem, alpha, theta, nullptr, errors, m_work, nullptr, m_chunk_states, nullptr, y,
        seq_len, d, chunk_size, chunk_idx, m_norm_max);
    check_launch("delta_phase2_forward_f32_cuda");
}

void titans_phase2_forward_f32_cuda(const float* k_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* eta, const float* errors, float* m_work, float* s_work,
    float* m_chunk_states, float* s_chunk_states, float* y, int32_t seq_len, int32_t d,
    int32_t batch_size, int32_t chunk_size, int32_t chunk_idx, float m_norm_max)
{
    if (!valid_dims("titans_phase2_forward_f32_cuda", seq_len, d, batch_size) || batch_size == 0) return;
    if (chunk_size <= 0 || chunk_idx < 0) { record_status(NLH_ERR_INVALID_ARG, "titans_phase2_forward_f32_cuda", "bad chunk"); return; }
    const size_t smem = gen_fwd_smem(d);
    if (smem > 48 * 1024) cudaFuncSetAttribute(gen_phase2_fwd_kernel<RULE_TITANS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gen_phase2_fwd_kernel<RULE_TITANS><<<batch_size, GEN_THREADS, smem, current_stream()>>>(
        k_mem, q_mem, alpha, theta, eta, errors, m_work, s_work, m_chunk_states, s_chunk_states, y,
        seq_len, d, chunk_size, chunk_idx, m_norm_max);
    check_launch("titans_phase2_forward_f32_cuda");
}

void delta_phase2_backward_f32_cuda(const float* k_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* errors, const float* m_chunk_states, const float* d_y,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_M,
    float* d_M0, float* m_recompute, int32_t seq_len, int32_t d, int32_t batch_size,
    int32_t chunk_size, int32_t chunk_idx, float m_norm_max)
{
    if (!valid_dims("delta_phase2_backward_f32_cuda", seq_len, d, batch_size) || batch_size == 0) return;
    if (chunk_size <= 0 || chunk_idx < 0) { record_status(NLH_ERR_INVALID_ARG, "delta_phase2_backward_f32_cuda", "bad chunk"); return; }
    const size_t smem = gen_bwd_smem(d);
    if (smem > 48 * 1024) cudaFuncSetAttribute(gen_phase2_bwd_kernel<RULE_DELTA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gen_phase2_bwd_kernel<RULE_DELTA><<<batch_size, GEN_THREADS, smem, current_stream()>>>(
        k_mem, q_mem, alpha, theta, nullptr, errors, m_chunk_states, nullptr, d_y, d_k_mem, d_v_mem,
        d_q_mem, d_alpha, d_theta, nullptr, d_M, nullptr, d_M0, m_recompute, nullptr, seq_len, d,
        chunk_size, chunk_idx, m_norm_max);
    check_launch("delta_phase2_backward_f32_cuda");
}

void titans_phase2_backward_f32_cuda(const float* k_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* eta, const float* errors, const float* m_chunk_states,
    const float* s_chunk_states, const float* d_y, float* d_k_mem, float* d_v_mem,
    float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta, float* d_M, float* d_S,
    float* d_M0, float* m_recompute, float* s_recompute, int32_t seq_len, int32_t d,
    int32_t batch_size, int32_t chunk_size, int32_t chunk_idx, float m_norm_max)
{
    if (!valid_dims("titans_phase2_backward_f32_cuda", seq_len, d, batch_size) || batch_size == 0) return;
    if (chunk_size <= 0 || chunk_idx < 0) { record_status(NLH_ERR_INVALID_ARG, "titans_phase2_backward_f32_cuda", "bad chunk"); return; }
    const size_t smem = gen_bwd_smem(d);
    if (smem > 48 * 1024) cudaFuncSetAttribute(gen_phase2_bwd_kernel<RULE_TITANS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gen_phase2_bwd_kernel<RULE_TITANS><<<batch_size, GEN_THREADS, smem, current_stream()>>>(
        k_mem, q_mem, alpha, theta, eta, errors, m_chunk_states, s_chunk_states, d_y, d_k_mem,
        d_v_mem, d_q_mem, d_alpha, d_theta, d_eta, d_M, d_S, d_M0, m_recompute, s_recompute,
        seq_len, d, chunk_size, chunk_idx, m_norm_max);
    check_launch("titans_phase2_backward_f32_cuda");
}

void m_norm_clamp_f32_cuda(float* m, int32_t d, float m_norm_max)
{
    m_norm_clamp_batch_f32_cuda(m, d, 1, m_norm_max);
}

void m_norm_clamp_batch_f32_cuda(float* m, int32_t d, int32_t batch_size, float m_norm_max)
{
    if (!m_norm_enabled(m_norm_max) || batch_size <= 0 || d <= 0) return;
    m_norm_clamp_kernel<<<batch_size, GEN_THREADS, 0, current_stream()>>>(m, (size_t)d * d,
                                                                        m_norm_max);
    check_launch("m_norm_clamp_batch_f32_cuda");
}

// ───────────────────────── fused forwards ─────────────────────────────────
void dgd_fused_forward_f32_cuda(float* k_mem, const float* v_mem, float* q_mem,
    const float* w_alpha, const float* b_alpha_ptr, const float* w_theta,
    const float* b_theta_ptr, float alpha_floor, float alpha_ceil, float theta_floor,
    float theta_ceil, const float* m_initial, float* m_states, float* y, float* alpha_out,
    float* theta_out, float* k_norms_out, float* q_norms_out, int32_t seq_len, int32_t d,
    int32_t batch_size, float error_clip)
{
    if (!valid_dims("dgd_fused_forward_f32_cuda", seq_len, d, batch_size) || batch_size == 0) return;
    const long long n_tok = (long long)batch_size * seq_len;
    if (n_tok > 0) {
        fused_prep_kernel<<<(unsigned)((n_tok + 7) / 8), 256, 0, current_stream()>>>(
            k_mem, v_mem, q_mem, w_alpha, b_alpha_ptr, w_theta, b_theta_ptr, nullptr, nullptr,
            alpha_floor, alpha_ceil, theta_floor, theta_ceil, alpha_out, theta_out, nullptr,
            k_norms_out, q_norms_out, n_tok, d);
        if (!check_launch("dgd_fused_forward_f32_cuda(prep)")) return;
    }
    run_forward(RULE_DELTA, fwd_args(k_mem, v_mem, q_mem, alpha_out, theta_out, nullptr, m_initial,
        nullptr, m_states, nullptr, y, seq_len, d, batch_size, seq_len, (long long)d * d,
        (long long)(seq_len + 1) * d * d, STORE_ALL, 0, 0, error_clip, 0.0f),
        "dgd_fused_forward_f32_cuda");
}

void titans_fused_forward_f32_cuda(float* k_mem, const float* v_mem, float* q_mem,
    const float* w_alpha, const float* b_alpha_ptr, const float* w_theta,
    const float* b_theta_ptr, const float* w_eta, const float* b_eta_ptr, float alpha_floor,
    float alpha_ceil, float theta_floor, float theta_ceil, const float* m_initial,
    const float* s_initial, float* m_states, float* s_states, float* y, float* alpha_out,
    float* theta_out, float* eta_out, float* k_norms_out, float* q_norms_out, int32_t seq_len,
    int32_t d, int32_t batch_size, float error_clip, float m_norm_max)
{
    if (!valid_dims("titans_fused_forward_f32_cuda", seq_len, d, batch_size) || batch_size == 0) return;
    const long long n_tok = (long long)batch_size * seq_len;
    if (n_tok > 0) {
        fused_prep_kernel<<<(unsigned)((n_tok + 7) / 8), 256, 0, current_stream()>>>(
            k_mem, v_mem, q_mem, w_alpha, b_alpha_ptr, w_theta, b_theta_ptr, w_eta, b_eta_ptr,
            alpha_floor, alpha_ceil, theta_floor, theta_ceil, alpha_out, theta_out, eta_out,
            k_norms_out, q_norms_out, n_tok, d);
        if (!check_launch("titans_fused_forward_f32_cuda(prep)")) return;
    }
    run_forward(RULE_TITANS, fwd_args(k_mem, v_mem, q_mem, alpha_out, theta_out, eta_out, m_initial,
        s_initial, m_states, s_states, y, seq_len, d, batch_size, seq_len, (long long)d * d,
        (long long)(seq_len + 1) * d * d, STORE_ALL, 0, 0, error_clip, m_norm_max),
        "titans_fused_forward_f32_cuda");
}

// ───────────────────────── additive training path ─────────────────────────
int32_t nlh_rule_forward(int32_t rule, const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_ckpt, float* s_ckpt, float* y, int32_t seq_len, int32_t d,
    int32_t batch_size, int32_t interval, int32_t chunk_size, float error_clip,
    float m_norm_max)
{
    if (interval <= 0 || chunk_size < 0 || (chunk_size > 0 && chunk_size != interval && interval != 1))
        return NLH_ERR_INVALID_ARG;
    if (rule == RULE_HEBBIAN && chunk_size > 0) return NLH_ERR_INVALID_ARG;
    const int frozen = chunk_size > 0 ? 1 : 0;
    if (frozen && interval == 1 && chunk_size > 1) {
        // frozen rule, every state stored: m_ckpt [B, S+1, d*d]; s_ckpt may be NULL (Titans)
        if (rule != RULE_TITANS || !fast_common_ok(d, error_clip, m_norm_max)) {
            record_status(NLH_ERR_UNSUPPORTED, "nlh_rule_forward",
                          "full-trajectory frozen mode: Titans, head_dim 32/64, no clip/projection");
            return NLH_ERR_UNSUPPORTED;
        }
        return run_forward(rule, fwd_args(k_mem, v_mem, q_mem, alpha, theta, eta, m_initial, s_initial,
            m_ckpt, s_ckpt, y, seq_len, d, batch_size, seq_len, (long long)d * d,
            (long long)(seq_len + 1) * d * d, STORE_ALL, chunk_size, 1, error_clip, m_norm_max),
            "nlh_rule_forward");
    }
    return run_forward(rule, fwd_args(k_mem, v_mem, q_mem, alpha, theta, eta, m_initial, s_initial,
        m_ckpt, s_ckpt, y, seq_len, d, batch_size, seq_len, (long long)d * d,
        ckpt_slots(seq_len, interval) * d * d, frozen ? STORE_CHUNK : STORE_CKPT, interval, frozen,
        error_clip, m_norm_max), "nlh_rule_forward");
}

int32_t nlh_rule_backward(int32_t rule, const float* k_mem, const float* v_mem,
    const float* q_mem, const float* alpha, const float* theta, const float* eta,
    const float* m_ckpt, const float* s_ckpt, const float* d_y, float* d_k_mem, float* d_v_mem,
    float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta, float* d_m_initial,
    float* d_s_initial, int32_t seq_len, int32_t d, int32_t batch_size, int32_t interval,
    int32_t chunk_size, float error_clip, float m_norm_max)
{
    if (interval <= 0 || chunk_size < 0 || (chunk_size > 0 && chunk_size != interval && interval != 1))
        return NLH_ERR_INVALID_ARG;
    if (rule == RULE_HEBBIAN && chunk_size > 0) return NLH_ERR_INVALID_ARG;
    const int frozen = chunk_size > 0 ? 1 : 0;
    if (frozen && interval == 1 && chunk_size > 1) {
        // frozen rule on a full M trajectory: streamed, nothing recomputed (s_ckpt is not read)
        const char* where = "nlh_rule_backward";
        if (!valid_dims(where, seq_len, d, batch_size)) return NLH_ERR_INVALID_ARG;
        if (batch_size == 0) return NLH_OK;
        BwdArgs a = bwd_args(k_mem, v_mem, q_mem, alpha, theta, eta, m_ckpt, nullptr, d_y, nullptr, nullptr,
            d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, d_eta, d_m_initial, d_s_initial, seq_len, d,
            batch_size, 0, seq_len, (long long)(seq_len + 1) * d * d, 1, chunk_size, 0, error_clip, m_norm_max);
        const bool al = aligned16(a.k) && aligned16(a.v) && aligned16(a.q) && aligned16(a.d_y) && aligned16(a.d_k) &&
                        aligned16(a.d_v) && aligned16(a.d_q) && aligned16(a.m_traj) &&
                        aligned16(a.d_m_out) && aligned16(a.d_s_out);
        if (rule != RULE_TITANS || !fast_common_ok(d, error_clip, m_norm_max) || !al || ((d_m_initial == nullptr) != (d_s_initial == nullptr))) {
            record_status(NLH_ERR_UNSUPPORTED, where,
                          "full-trajectory frozen mode: Titans, head_dim 32/64, no clip/projection, 16-byte aligned buffers");
            return NLH_ERR_UNSUPPORTED;
        }
        cudaStream_t st = current_stream();
        if (d == 64) frozen_stream_bwd_launch<64>(a, st); else frozen_stream_bwd_launch<32>(a, st);
        return check_launch(where) ? NLH_OK : NLH_ERR_CUDA;
    }
    return run_backward(rule, bwd_args(k_mem, v_mem, q_mem, alpha, theta, eta, m_ckpt, s_ckpt, d_y,
        nullptr, nullptr, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, d_eta, d_m_initial,
        d_s_initial, seq_len, d, batch_size, 0, seq_len, ckpt_slots(seq_len, interval) * d * d,
        frozen, interval, 0, error_clip, m_norm_max), "nlh_rule_backward");
}

int32_t nlh_bulk_timeout_flag(void)
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_bulk_timeout, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

}  // extern "C"
