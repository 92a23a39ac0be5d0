// Host-slice dispatch layer: the compiled counterpart of the reference's `*_dispatch` functions
// (core/src/dispatch.rs:378-460 SWA, :746-1213 memory rules), which its kernel tests call with
// host slices (core/tests/test_cuda_*.rs). Same argument order and meaning; pointers are HOST
// pointers, one sequence (no batch argument, as in the reference); every entry uploads, runs the
// drop-in kernel entry, downloads and synchronises, returning an int32 status instead of
// panicking. SWA converts q,k,v to bf16 on the device like dispatch.rs:478-560 does on the host;
// its backward accumulates into d_q,d_k,d_v (caller pre-zeroes, dispatch.rs:404-407).
#include <cuda_bf16.h>

#include "host_staging.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {

__global__ void hd_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = __float2bfloat16(src[i]);
}
__global__ void hd_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = __bfloat162float(src[i]);
}
static unsigned hd_grid(long long n) { long long g = (n + 255) / 256; return (unsigned)(g < 1 ? 1 : (g > 4096 ? 4096 : g)); }

static int hd_fail(const char* where, int code, const char* detail)
{
    record_status(code, where, detail);
    return code;
}
static int hd_finish(const char* where, cudaStream_t st)
{
    if (nlh_last_status() != NLH_OK) return nlh_last_status();
    if (cudaStreamSynchronize(st) != cudaSuccess) return hd_fail(where, NLH_ERR_CUDA, "stream synchronisation failed");
    return NLH_OK;
}

// Shared body of the memory-rule forwards. rule: 0 delta, 1 titans, 2 hebbian, 3 dgd.
static int rule_forward(const char* where, int rule, const float* k, const float* v, const float* q,
                        const float* alpha, const float* theta, const float* eta, const float* m_initial,
                        const float* s_initial, float* m_states, float* s_states, float* y,
                        long long seq, long long d, float clip, float m_norm_max)
{
    if (seq <= 0 || d <= 0 || !k || !v || !q || !alpha || !m_initial || !m_states || !y)
        return hd_fail(where, NLH_ERR_INVALID_ARG, "bad dimensions or NULL pointer");
    // per-rule required inputs: every rule but Hebbian reads theta, Titans also eta and s_initial
    if ((rule != 2 && !theta) || (rule == 1 && (!eta || !s_initial)))
        return hd_fail(where, NLH_ERR_INVALID_ARG, "NULL gate or initial-state pointer for this rule");
    cudaStream_t st = current_stream();
    Staging sg;
    const long long sd = seq * d, dd = d * d, tr = (seq + 1) * dd;
    float *dk = sg.upload(k, sd, st), *dv = sg.upload(v, sd, st), *dq = sg.upload(q, sd, st);
    float* dal = sg.upload(alpha, seq, st);
    float* dth = theta ? sg.upload(theta, seq, st) : nullptr;
    float* det = eta ? sg.upload(eta, seq, st) : nullptr;
    float* dm0 = sg.upload(m_initial, dd, st);
    float* ds0 = s_initial ? sg.upload(s_initial, dd, st) : nullptr;
    float* dms = sg.empty(tr);
    float* dss = s_states ? sg.empty(tr) : nullptr;
    float* dy = sg.empty(sd);
    if (!sg.ok) return hd_fail(where, NLH_ERR_CUDA, "device staging failed");
    nlh_clear_status();
    const int S = (int)seq, D = (int)d;
    if (rule == 0) delta_forward_f32_cuda(dk, dv, dq, dal, dth, dm0, dms, dy, S, D, 1, S, D * D, clip, m_norm_max);
    else if (rule == 1) titans_forward_f32_cuda(dk, dv, dq, dal, dth, det, dm0, ds0, dms, dss, dy, S, D, 1, S, D * D, clip, m_norm_max);
    else if (rule == 2) hebbian_forward_f32_cuda(dk, dv, dq, dal, dm0, dms, dy, S, D, 1, S, D * D);
    else dgd_forward_f32_cuda(dk, dv, dq, dal, dth, dm0, dms, dy, S, D, 1, S, D * D, clip);
    if (nlh_last_status() != NLH_OK) return nlh_last_status();
    if (!download(m_states, dms, tr, st) || !download(y, dy, sd, st) || (s_states && !download(s_states, dss, tr, st)))
        return hd_fail(where, NLH_ERR_CUDA, "download failed");
    return hd_finish(where, st);
}

static int rule_backward(const char* where, int rule, const float* k, const float* v, const float* q,
                         const float* alpha, const float* theta, const float* eta, const float* m_states,
                         const float* s_states, const float* d_y, float* d_k, float* d_v, float* d_q,
                         float* d_alpha, float* d_theta, float* d_eta, float* d_m_initial,
                         float* d_s_initial, long long seq, long long d, float clip)
{
    if (seq <= 0 || d <= 0 || !k || !v || !q || !alpha || !m_states || !d_y || !d_k || !d_v || !d_q ||
        !d_alpha || !d_m_initial)
        return hd_fail(where, NLH_ERR_INVALID_ARG, "bad dimensions or NULL pointer");
    // per-rule required gates and gate gradients (Hebbian has neither theta nor eta)
    if ((rule != 2 && (!theta || !d_theta)) || (rule == 1 && (!eta || !d_eta || !s_states || !d_s_initial)))
        return hd_fail(where, NLH_ERR_INVALID_ARG, "NULL gate, gate-gradient or state pointer for this rule");
    cudaStream_t st = current_stream();
    Staging sg;
    const long long sd = seq * d, dd = d * d, tr = (seq + 1) * dd;
    float *dk = sg.upload(k, sd, st), *dv = sg.upload(v, sd, st), *dq = sg.upload(q, sd, st);
    float* dal = sg.upload(alpha, seq, st);
    float* dth = theta ? sg.upload(theta, seq, st) : nullptr;
    float* det = eta ? sg.upload(eta, seq, st) : nullptr;
    float* dms = sg.upload(m_states, tr, st);
    float* dss = s_states ? sg.upload(s_states, tr, st) : nullptr;
    float* ddy = sg.upload(d_y, sd, st);
    float *gk = sg.zeros(sd, st), *gv = sg.zeros(sd, st), *gq = sg.zeros(sd, st);
    float *ga = sg.zeros(seq, st), *gt = sg.zeros(seq, st), *ge = sg.zeros(seq, st);
    float *gm = sg.zeros(dd, st), *gs = sg.zeros(dd, st);
    if (!sg.ok) return hd_fail(where, NLH_ERR_CUDA, "device staging failed");
    nlh_clear_status();
    const int S = (int)seq, D = (int)d;
    if (rule == 0) delta_backward_f32_cuda(dk, dv, dq, dal, dth, dms, ddy, gk, gv, gq, ga, gt, gm, S, D, 1, clip);
    else if (rule == 1) titans_backward_f32_cuda(dk, dv, dq, dal, dth, det, dms, dss, ddy, gk, gv, gq, ga, gt, ge, gm, gs, S, D, 1, clip);
    else if (rule == 2) hebbian_backward_f32_cuda(dk, dv, dq, dal, dms, ddy, gk, gv, gq, ga, gm, S, D);
    else dgd_backward_f32_cuda(dk, dv, dq, dal, dth, dms, ddy, gk, gv, gq, ga, gt, gm, S, D, clip);
    if (nlh_last_status() != NLH_OK) return nlh_last_status();
    bool ok = download(d_k, gk, sd, st) && download(d_v, gv, sd, st) && download(d_q, gq, sd, st) &&
              download(d_alpha, ga, seq, st) && download(d_m_initial, gm, dd, st);
    if (d_theta) ok = ok && download(d_theta, gt, seq, st);
    if (d_eta) ok = ok && download(d_eta, ge, seq, st);
    if (d_s_initial) ok = ok && download(d_s_initial, gs, dd, st);
    if (!ok) return hd_fail(where, NLH_ERR_CUDA, "download failed");
    return hd_finish(where, st);
}

}  // namespace nlh

using namespace nlh;

extern "C" {

int32_t nlh_delta_forward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int64_t seq_len, int64_t d, float error_clip, float m_norm_max)
{
    return rule_forward("nlh_delta_forward_dispatch", 0, k_mem, v_mem, q_mem, alpha, theta, nullptr, m_initial,
                        nullptr, m_states, nullptr, y, seq_len, d, error_clip, m_norm_max);
}
int32_t nlh_delta_backward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y, float* d_k_mem,
    float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_m_initial, int64_t seq_len,
    int64_t d, float error_clip)
{
    return rule_backward("nlh_delta_backward_dispatch", 0, k_mem, v_mem, q_mem, alpha, theta, nullptr, m_states,
                         nullptr, d_y, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, nullptr, d_m_initial, nullptr,
                         seq_len, d, error_clip);
}
int32_t nlh_titans_forward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial,
    const float* s_initial, float* m_states, float* s_states, float* y, int64_t seq_len, int64_t d,
    float error_clip, float m_norm_max)
{
    if (!theta || !eta || !s_initial || !s_states) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_titans_forward_dispatch", "NULL pointer");
        return NLH_ERR_INVALID_ARG;
    }
    return rule_forward("nlh_titans_forward_dispatch", 1, k_mem, v_mem, q_mem, alpha, theta, eta, m_initial,
                        s_initial, m_states, s_states, y, seq_len, d, error_clip, m_norm_max);
}
int32_t nlh_titans_backward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_states,
    const float* s_states, const float* d_y, float* d_k_mem, float* d_v_mem, float* d_q_mem,
    float* d_alpha, float* d_theta, float* d_eta, float* d_m_initial, float* d_s_initial,
    int64_t seq_len, int64_t d, float error_clip)
{
    if (!theta || !eta || !s_states || !d_theta || !d_eta || !d_s_initial) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_titans_backward_dispatch", "NULL pointer");
        return NLH_ERR_INVALID_ARG;
    }
    return rule_backward("nlh_titans_backward_dispatch", 1, k_mem, v_mem, q_mem, alpha, theta, eta, m_states,
                         s_states, d_y, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, d_eta, d_m_initial,
                         d_s_initial, seq_len, d, error_clip);
}
int32_t nlh_hebbian_forward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_initial, float* m_states, float* y, int64_t seq_len, int64_t d)
{
    return rule_forward("nlh_hebbian_forward_dispatch", 2, k_mem, v_mem, q_mem, alpha, nullptr, nullptr,
                        m_initial, nullptr, m_states, nullptr, y, seq_len, d, 0.0f, 0.0f);
}
int32_t nlh_hebbian_backward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* m_states, const float* d_y, float* d_k_mem, float* d_v_mem,
    float* d_q_mem, float* d_alpha, float* d_m_initial, int64_t seq_len, int64_t d)
{
    return rule_backward("nlh_hebbian_backward_dispatch", 2, k_mem, v_mem, q_mem, alpha, nullptr, nullptr,
                         m_states, nullptr, d_y, d_k_mem, d_v_mem, d_q_mem, d_alpha, nullptr, nullptr,
                         d_m_initial, nullptr, seq_len, d, 0.0f);
}
int32_t nlh_dgd_forward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_initial, float* m_states, float* y,
    int64_t seq_len, int64_t d, float error_clip)
{
    return rule_forward("nlh_dgd_forward_dispatch", 3, k_mem, v_mem, q_mem, alpha, theta, nullptr, m_initial,
                        nullptr, m_states, nullptr, y, seq_len, d, error_clip, 0.0f);
}
int32_t nlh_dgd_backward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* m_states, const float* d_y, float* d_k_mem,
    float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_m_initial, int64_t seq_len,
    int64_t d, float error_clip)
{
    return rule_backward("nlh_dgd_backward_dispatch", 3, k_mem, v_mem, q_mem, alpha, theta, nullptr, m_states,
                         nullptr, d_y, d_k_mem, d_v_mem, d_q_mem, d_alpha, d_theta, nullptr, d_m_initial, nullptr,
                         seq_len, d, error_clip);
}

// Titans LMM with a two-layer MLP memory, host slices in and out: titans_mlp_forward_cuda /
// titans_mlp_backward_cuda (core/src/dispatch.rs:897-1070), which, unlike the other host-slice
// functions, take a batch. d_m_initial / d_s_initial [state_size] are the sums over the batch.
int32_t nlh_titans_mlp_forward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_initial, const float* s_initial,
    float* m_states, float* s_states, float* y, int64_t seq_len, int64_t d, int64_t d_hidden, int64_t batch_size,
    int32_t activation, float m_norm_max)
{
    const char* where = "nlh_titans_mlp_forward_dispatch";
    if (seq_len <= 0 || d <= 0 || d_hidden <= 0 || batch_size <= 0 || !k_mem || !v_mem || !q_mem || !alpha || !theta ||
        !eta || !m_initial || !s_initial || !m_states || !s_states || !y)
        return hd_fail(where, NLH_ERR_INVALID_ARG, "bad dimensions or NULL pointer");
    const long long ss = 2 * d * d_hidden + d_hidden + d, sd = batch_size * seq_len * d, sg_ = batch_size * seq_len;
    const long long tr = batch_size * (seq_len + 1) * ss;
    if ((seq_len + 1) * ss > 0x7fffffffLL) return hd_fail(where, NLH_ERR_INVALID_ARG, "m_stride does not fit the int32 argument of the entry");
    cudaStream_t st = current_stream();
    Staging sg;
    float *dk = sg.upload(k_mem, sd, st), *dv = sg.upload(v_mem, sd, st), *dq = sg.upload(q_mem, sd, st);
    float *dal = sg.upload(alpha, sg_, st), *dth = sg.upload(theta, sg_, st), *det = sg.upload(eta, sg_, st);
    float *dm0 = sg.upload(m_initial, batch_size * ss, st), *ds0 = sg.upload(s_initial, batch_size * ss, st);
    float *dms = sg.empty(tr), *dss = sg.empty(tr), *dy = sg.empty(sd);
    if (!sg.ok) return hd_fail(where, NLH_ERR_CUDA, "device staging failed");
    nlh_clear_status();
    titans_mlp_forward_f32_cuda(dk, dv, dq, dal, dth, det, dm0, ds0, dms, dss, dy, (int)seq_len, (int)d, (int)d_hidden,
                                (int)batch_size, (int)(seq_len * d), (int)((seq_len + 1) * ss), activation, m_norm_max);
    if (nlh_last_status() != NLH_OK) return nlh_last_status();
    if (!download(m_states, dms, tr, st) || !download(s_states, dss, tr, st) || !download(y, dy, sd, st))
        return hd_fail(where, NLH_ERR_CUDA, "download failed");
    return hd_finish(where, st);
}
int32_t nlh_titans_mlp_backward_dispatch(const float* k_mem, const float* v_mem, const float* q_mem,
    const float* alpha, const float* theta, const float* eta, const float* m_states, const float* s_states,
    const float* d_y, float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta,
    float* d_m_initial, float* d_s_initial, int64_t seq_len, int64_t d, int64_t d_hidden, int64_t batch_size,
    int32_t activation, float m_norm_max)
{
    const char* where = "nlh_titans_mlp_backward_dispatch";
    if (seq_len <= 0 || d <= 0 || d_hidden <= 0 || batch_size <= 0 || !k_mem || !v_mem || !q_mem || !alpha || !theta ||
        !eta || !m_states || !s_states || !d_y || !d_k_mem || !d_v_mem || !d_q_mem || !d_alpha || !d_theta || !d_eta ||
        !d_m_initial || !d_s_initial)
        return hd_fail(where, NLH_ERR_INVALID_ARG, "bad dimensions or NULL pointer");
    const long long ss = 2 * d * d_hidden + d_hidden + d, sd = batch_size * seq_len * d, sg_ = batch_size * seq_len;
    const long long tr = batch_size * (seq_len + 1) * ss;
    if ((seq_len + 1) * ss > 0x7fffffffLL) return hd_fail(where, NLH_ERR_INVALID_ARG, "m_stride does not fit the int32 argument of the entry");
    cudaStream_t st = current_stream();
    Staging sg;
    float *dk = sg.upload(k_mem, sd, st), *dv = sg.upload(v_mem, sd, st), *dq = sg.upload(q_mem, sd, st);
    float *dal = sg.upload(alpha, sg_, st), *dth = sg.upload(theta, sg_, st), *det = sg.upload(eta, sg_, st);
    float *dms = sg.upload(m_states, tr, st), *dss = sg.upload(s_states, tr, st), *ddy = sg.upload(d_y, sd, st);
    float *gk = sg.empty(sd), *gv = sg.empty(sd), *gq = sg.empty(sd);
    float *ga = sg.empty(sg_), *gt = sg.empty(sg_), *ge = sg.empty(sg_);
    float *gm = sg.zeros(ss, st), *gs = sg.zeros(ss, st);
    if (!sg.ok) return hd_fail(where, NLH_ERR_CUDA, "device staging failed");
    nlh_clear_status();
    titans_mlp_backward_f32_cuda(dk, dv, dq, dal, dth, det, dms, dss, ddy, gk, gv, gq, ga, gt, ge, gm, gs, (int)seq_len,
                                 (int)d, (int)d_hidden, (int)batch_size, (int)(seq_len * d), (int)((seq_len + 1) * ss),
                                 activation, m_norm_max);
    if (nlh_last_status() != NLH_OK) return nlh_last_status();
    const bool ok = download(d_k_mem, gk, sd, st) && download(d_v_mem, gv, sd, st) && download(d_q_mem, gq, sd, st) &&
                    download(d_alpha, ga, sg_, st) && download(d_theta, gt, sg_, st) && download(d_eta, ge, sg_, st) &&
                    download(d_m_initial, gm, ss, st) && download(d_s_initial, gs, ss, st);
    if (!ok) return hd_fail(where, NLH_ERR_CUDA, "download failed");
    return hd_finish(where, st);
}

int32_t nlh_swa_forward_dispatch(const float* q, const float* k, const float* v, float* out,
    float* attn_weights, int64_t seq_len, int64_t num_heads, int64_t head_dim, int64_t window_size)
{
    const char* where = "nlh_swa_forward_dispatch";
    if (seq_len <= 0 || num_heads <= 0 || head_dim <= 0 || window_size <= 0 || !q || !k || !v || !out)
        return hd_fail(where, NLH_ERR_INVALID_ARG, "bad dimensions or NULL pointer");
    cudaStream_t st = current_stream();
    Staging sg;
    const long long n = seq_len * num_heads * head_dim, nw = num_heads * seq_len * window_size;
    __nv_bfloat16* h16[3];
    const float* src[3] = {q, k, v};
    for (int i = 0; i < 3; i++) {
        float* f = sg.upload(src[i], n, st);
        h16[i] = (__nv_bfloat16*)sg.alloc((size_t)n * 2);
        if (!sg.ok) return hd_fail(where, NLH_ERR_CUDA, "device staging failed");
        hd_f32_to_bf16_kernel<<<hd_grid(n), 256, 0, st>>>(f, h16[i], n);
    }
    __nv_bfloat16* o16 = (__nv_bfloat16*)sg.alloc((size_t)n * 2);
    __nv_bfloat16* w16 = attn_weights ? (__nv_bfloat16*)sg.alloc((size_t)nw * 2) : nullptr;
    float* of = sg.empty(n);
    float* wf = attn_weights ? sg.empty(nw) : nullptr;
    if (!sg.ok) return hd_fail(where, NLH_ERR_CUDA, "device staging failed");
    nlh_clear_status();
    swa_forward_f32_cuda((const uint16_t*)h16[0], (const uint16_t*)h16[1], (const uint16_t*)h16[2], (uint16_t*)o16,
                         (uint16_t*)w16, (int)seq_len, (int)num_heads, (int)head_dim, (int)window_size, 1, 0);
    if (nlh_last_status() != NLH_OK) return nlh_last_status();
    hd_bf16_to_f32_kernel<<<hd_grid(n), 256, 0, st>>>(o16, of, n);
    if (attn_weights) hd_bf16_to_f32_kernel<<<hd_grid(nw), 256, 0, st>>>(w16, wf, nw);
    if (!check_launch(where)) return NLH_ERR_CUDA;
    if (!download(out, of, n, st) || (attn_weights && !download(attn_weights, wf, nw, st)))
        return hd_fail(where, NLH_ERR_CUDA, "download failed");
    return hd_finish(where, st);
}

int32_t nlh_swa_backward_dispatch(const float* q, const float* k, const float* v, const float* attn_weights,
    const float* d_attn_out, float* d_q, float* d_k, float* d_v, int64_t seq_len, int64_t num_heads,
    int64_t head_dim, int64_t window_size)
{
    const char* where = "nlh_swa_backward_dispatch";
    (void)attn_weights;   // recomputed from q and k on the device
    if (seq_len <= 0 || num_heads <= 0 || head_dim <= 0 || window_size <= 0 || !q || !k || !v ||
        !d_attn_out || !d_q || !d_k || !d_v)
        return hd_fail(where, NLH_ERR_INVALID_ARG, "bad dimensions or NULL pointer");
    cudaStream_t st = current_stream();
    Staging sg;
    const long long n = seq_len * num_heads * head_dim;
    __nv_bfloat16* h16[3];
    const float* src[3] = {q, k, v};
    for (int i = 0; i < 3; i++) {
        float* f = sg.upload(src[i], n, st);
        h16[i] = (__nv_bfloat16*)sg.alloc((size_t)n * 2);
        if (!sg.ok) return hd_fail(where, NLH_ERR_CUDA, "device staging failed");
        hd_f32_to_bf16_kernel<<<hd_grid(n), 256, 0, st>>>(f, h16[i], n);
    }
    float* dout = sg.upload(d_attn_out, n, st);
    // the reference accumulates into caller-zeroed gradients: start from the caller's values
    float *gk = sg.upload(d_k, n, st), *gv = sg.upload(d_v, n, st);
    float* gq_new = sg.zeros(n, st);
    if (!sg.ok || !check_launch(where)) return hd_fail(where, NLH_ERR_CUDA, "device staging failed");
    nlh_clear_status();
    // d_q of the drop-in entry is overwritten, d_k/d_v are added into
    swa_backward_f32_cuda((const uint16_t*)h16[0], (const uint16_t*)h16[1], (const uint16_t*)h16[2], nullptr, dout,
                          gq_new, gk, gv, (int)seq_len, (int)num_heads, (int)head_dim, (int)window_size, 1, 0);
    if (nlh_last_status() != NLH_OK) return nlh_last_status();
    std::vector<float> tmp((size_t)n);
    if (!download(tmp.data(), gq_new, n, st) || !download(d_k, gk, n, st) || !download(d_v, gv, n, st))
        return hd_fail(where, NLH_ERR_CUDA, "download failed");
    const int rc = hd_finish(where, st);
    if (rc == NLH_OK)
        for (long long i = 0; i < n; i++) d_q[i] += tmp[(size_t)i];
    return rc;
}

}  // extern "C"
