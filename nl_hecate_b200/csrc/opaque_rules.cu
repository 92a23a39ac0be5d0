// Rule-level opaque-VJP adapters on the GPU: the backward of one whole memory-rule block
// `(embedded, level_params_flat) -> y` as the reference's Wengert tape records it
// (OpaqueKey::{DeltaRule, TitansLMM, HebbianRule}, core/src/tape.rs:100-104).
//
// Function replaced: {delta_rule,titans_lmm,hebbian}_opaque_backward, core/src/opaque_adapters.rs
// :306-381, :402-590, :593-628, i.e. DeltaRule / TitansLMM / HebbianRule::step_backward
// (core/src/delta_rule.rs:420-640, titans_lmm.rs:1535-1764 + projection_backward :515-567,
// hebbian_rule.rs:183-300) on the buffers record_on_tape saved (opaque_adapters.rs:1180-1385):
//   Delta   saved = [meta(12), lp_flat, embedded, m_states, k_mem, v_mem, q_mem, concat_kv, alpha_pre,
//                    alpha, theta_pre, theta, error, grad_outer, y, k_norms, q_norms]
//   Titans  saved = [meta(16), lp_flat, embedded, m_states, s_states, k_mem, v_mem, q_mem, concat_kv,
//                    alpha_pre, alpha, theta_pre, theta, eta_pre, eta, error, grad_outer, y, k_norms,
//                    q_norms]
//   Hebbian saved = [meta(3), lp_flat, embedded, m_states, k_mem, v_mem, q_mem, concat_kv, alpha_pre,
//                    alpha, y]
// d_inputs[0] = d_embedded [seq*d]; d_inputs[1] = gradient of the flat parameter vector in the
// order of level_params_to_flat (opaque_adapters.rs:93-113): w_k_mem, w_v_mem, w_q_mem, w_alpha,
// b_alpha, w_theta, b_theta, w_eta, b_eta, then zeros up to its length.
//
// Steps on the device: (1) the rule's inner-loop backward kernel on the saved trajectory;
// (2) gate adjoints with the reference's straight-through clamp masks, gate -> k/v gradient and
// the L2-normalisation Jacobian; (3) gate weight gradients (a reduction over tokens);
// (4) projection backward: d W_{k|v|q} = d_kvq^T embedded and d_embedded = d_kvq [W_k; W_v; W_q]
// with the bf16-rounded weights the forward multiplied by (core/src/bf16.rs:54-115).
// Supported: identity feature map, L2 attentional bias, EMA / no momentum, linear memory, no
// conv1d — everything else returns NLH_ERR_UNSUPPORTED.
#include <cuda_bf16.h>

#include "host_staging.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {

__device__ __forceinline__ float orl_sigmoid(float x)
{
    if (x >= 15.0f) return 1.0f;
    if (x <= -15.0f) return 0.0f;
    return 1.0f / (1.0f + expf(-x));
}
__device__ __forceinline__ float orl_softplus(float x)
{
    if (x >= 15.0f) return x;
    if (x <= -15.0f) return 0.0f;
    return logf(1.0f + expf(x));
}

struct GateArgs {
    const float *k, *v, *q;                 // saved k_mem (normalised unless Hebbian), v_mem, q_mem  [s, d]
    const float *dk, *dv, *dq;              // from the inner-loop backward                            [s, d]
    const float *d_alpha, *d_theta, *d_eta; // [s]
    const float *alpha_pre, *alpha, *theta_pre, *theta, *eta;   // saved gates [s]
    const float *w_alpha, *w_theta, *w_eta; // [2d] each (device copies of the flat vector's slices)
    const float *k_norm, *q_norm;           // [s] or NULL (no normalisation)
    float *d_kvq;                           // [s, 3d]: d k_raw | d v | d q_raw
    float *dpre;                            // [s, 3]
    float a_lo, a_hi, t_lo, t_hi;
    int s, d, rule;                         // rule: 0 delta, 1 titans, 2 hebbian
};

// One CTA per token.
__global__ void __launch_bounds__(128) rule_gate_bwd_kernel(GateArgs a)
{
    __shared__ float red[32];
    const int t = blockIdx.x, d = a.d;
    const float al = a.alpha[t];
    float dp[3] = {0.f, 0.f, 0.f};
    {
        // alpha = sigmoid(alpha_pre) (clamped); Titans masks a clamped gate, Delta and Hebbian do not
        float mask = 1.0f;
        if (a.rule == 1) {
            const float raw = orl_sigmoid(a.alpha_pre[t]);
            mask = (raw <= a.a_lo || raw >= a.a_hi) ? 0.0f : 1.0f;
        }
        dp[0] = a.d_alpha[t] * al * (1.0f - al) * mask;
    }
    if (a.rule != 2) {
        // theta = softplus(theta_pre) clamped; Titans tests the raw value, Delta the saved (clamped) one
        const float tp = a.theta_pre[t];
        const float raw = (a.rule == 1) ? orl_softplus(tp) : a.theta[t];
        const float mask = (raw <= a.t_lo || raw >= a.t_hi) ? 0.0f : 1.0f;
        dp[1] = a.d_theta[t] * orl_sigmoid(tp) * mask;
    }
    if (a.rule == 1) {
        const float et = a.eta[t];
        dp[2] = a.d_eta[t] * et * (1.0f - et);
    }
    float dotk = 0.f, dotq = 0.f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const size_t o = (size_t)t * d + j;
        float gk = a.dk[o] + dp[0] * a.w_alpha[j];
        float gv = a.dv[o] + dp[0] * a.w_alpha[d + j];
        if (a.rule != 2) { gk += dp[1] * a.w_theta[j]; gv += dp[1] * a.w_theta[d + j]; }
        if (a.rule == 1) { gk += dp[2] * a.w_eta[j]; gv += dp[2] * a.w_eta[d + j]; }
        a.d_kvq[(size_t)t * 3 * d + j] = gk;            // provisional: normalisation Jacobian below
        a.d_kvq[(size_t)t * 3 * d + d + j] = gv;
        dotk += gk * a.k[o];
        dotq += a.dq[o] * a.q[o];
    }
    dotk = block_sum(dotk, red);
    dotq = block_sum(dotq, red);
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const size_t o = (size_t)t * d + j;
        float* row = a.d_kvq + (size_t)t * 3 * d;
        if (a.k_norm != nullptr) {
            // x_hat = x / max(||x||, 1e-8): d x = (g - x_hat (g . x_hat)) / ||x||  (core/src/tensor.rs:320-351)
            const float kn = a.k_norm[t], qn = a.q_norm[t];
            row[j] = (kn >= 1e-8f) ? (row[j] - a.k[o] * dotk) / kn : row[j] * 1e8f;
            row[2 * d + j] = (qn >= 1e-8f) ? (a.dq[o] - a.q[o] * dotq) / qn : a.dq[o] * 1e8f;
        } else {
            row[2 * d + j] = a.dq[o];
        }
    }
    if (threadIdx.x == 0) { a.dpre[t * 3 + 0] = dp[0]; a.dpre[t * 3 + 1] = dp[1]; a.dpre[t * 3 + 2] = dp[2]; }
}

// d w_g[j] = sum_t dpre[t][g] concat[t][j], d b_g = sum_t dpre[t][g], written into the flat
// gradient at offset base + g (2d + 1). One thread per (g, j), j = 2d is the bias.
__global__ void __launch_bounds__(128) rule_gate_wgrad_kernel(const float* __restrict__ dpre,
    const float* __restrict__ concat, float* __restrict__ d_flat, int s, int d, long long base)
{
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int per = 2 * d + 1;
    if (idx >= 3 * per) return;
    const int g = idx / per, j = idx - g * per;
    float acc = 0.f;
    for (int t = 0; t < s; t++) {
        const float p = dpre[t * 3 + g];
        acc += (j < 2 * d) ? p * concat[(size_t)t * 2 * d + j] : p;
    }
    d_flat[base + (long long)g * per + j] = acc;
}

__global__ void bf16_round_kernel(const float* __restrict__ src, float* __restrict__ dst, long long n)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = __bfloat162float(__float2bfloat16(src[i]));
}

// C[M,N] = A^T B (TA) or A B (!TA); fp32, 32x32 tiles through shared memory.
// TA:  A is [K, M] with leading dimension lda, B [K, N];  !TA: A is [M, K].
template <bool TA>
__global__ void __launch_bounds__(256) orl_sgemm_kernel(const float* __restrict__ A, int lda,
    const float* __restrict__ B, int ldb, float* __restrict__ C, int ldc, int M, int N, int K)
{
    __shared__ float As[32][33], Bs[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;        // 32 x 8
    const int m0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += 32) {
        for (int r = ty; r < 32; r += 8) {
            // As[kk][mm], Bs[kk][nn]
            if (TA) {
                const int kk = r, mm = tx;
                As[kk][mm] = (k0 + kk < K && m0 + mm < M) ? A[(size_t)(k0 + kk) * lda + m0 + mm] : 0.f;
            } else {
                const int mm = r, kk = tx;
                As[kk][mm] = (k0 + kk < K && m0 + mm < M) ? A[(size_t)(m0 + mm) * lda + k0 + kk] : 0.f;
            }
            const int kk = r, nn = tx;
            Bs[kk][nn] = (k0 + kk < K && n0 + nn < N) ? B[(size_t)(k0 + kk) * ldb + n0 + nn] : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; kk++) {
            const float b = Bs[kk][tx];
#pragma unroll
            for (int i = 0; i < 4; i++) acc[i] = fmaf(As[kk][ty + 8 * i], b, acc[i]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty + 8 * i, n = n0 + tx;
        if (m < M && n < N) C[(size_t)m * ldc + n] = acc[i];
    }
}

static int orl_fail(int code, const char* detail)
{
    record_status(code, "nlh_opaque_backward", detail);
    return code;
}

// rule: 0 delta, 1 titans, 2 hebbian. Host slices in, host slices out.
int opaque_rule_backward(int rule, int n_out, const float* const* d_outputs, const int64_t* out_len,
                         int n_saved, const float* const* saved, const int64_t* saved_len, int n_in,
                         float* const* d_inputs, const int64_t* in_len)
{
    const float* meta = saved[0];
    const long long ml = saved_len[0];
    const long long seq = (long long)meta[0], d = (long long)meta[1];
    if (seq <= 0 || d <= 0) return orl_fail(NLH_ERR_INVALID_ARG, "rule adapter: meta must hold seq > 0, d > 0");
    const long long sd = seq * d, dd = d * d, tr = (seq + 1) * dd, nflat = 3 * dd + 6 * d + 3;
    float a_lo = 0.f, a_hi = 1.f, t_lo = 0.f, t_hi = 3.402823466e38f;
    int base;     // index of m_states in saved
    int need;     // saved buffers required
    if (rule == 0) {
        if (ml < 12) return orl_fail(NLH_ERR_UNSUPPORTED, "DeltaRule: meta of an older tape format (no L2-norm buffers)");
        if (meta[2] != 2.0f || meta[6] != 0.0f || meta[ml - 1] != 0.0f)
            return orl_fail(NLH_ERR_UNSUPPORTED, "DeltaRule: only L2 bias, identity feature map, no conv1d are on the path");
        t_lo = meta[4]; t_hi = meta[5]; a_lo = meta[9]; a_hi = meta[10];
        base = 3; need = 17;
    } else if (rule == 1) {
        if (ml < 16) return orl_fail(NLH_ERR_UNSUPPORTED, "TitansLMM: meta of an older tape format");
        if (meta[2] != 2.0f || meta[7] != 0.0f || meta[ml - 1] != 0.0f || meta[12] >= 2.0f || meta[4] > 1.0f)
            return orl_fail(NLH_ERR_UNSUPPORTED,
                            "TitansLMM: only L2 bias, identity feature map, EMA momentum, linear memory, no conv1d are on the path");
        t_lo = meta[5]; t_hi = meta[6]; a_lo = meta[10]; a_hi = meta[11];
        base = 3; need = 20;
    } else {
        if (ml < 3 || meta[ml - 1] != 0.0f) return orl_fail(NLH_ERR_UNSUPPORTED, "HebbianRule: conv1d is not on the path");
        base = 3; need = 11;
    }
    if (n_saved < need || n_in < 2 || out_len[0] != sd || saved_len[1] < nflat || saved_len[2] != sd ||
        saved_len[base] != tr || in_len[0] != sd || in_len[1] < nflat)
        return orl_fail(NLH_ERR_INVALID_ARG, "rule adapter: buffer counts or lengths do not match meta (seq, d)");
    // positions inside saved
    const int i_s = (rule == 1) ? base + 1 : -1;
    const int i_k = (rule == 1) ? base + 2 : base + 1;
    const int i_cc = i_k + 3, i_ap = i_k + 4, i_a = i_k + 5;
    const int i_tp = (rule != 2) ? i_k + 6 : -1, i_t = (rule != 2) ? i_k + 7 : -1;
    const int i_e = (rule == 1) ? i_k + 9 : -1;
    const int i_kn = (rule == 0) ? 15 : (rule == 1 ? 18 : -1);
    for (int i = i_k; i < i_k + 3; i++)
        if (saved_len[i] != sd) return orl_fail(NLH_ERR_INVALID_ARG, "rule adapter: k/v/q_mem length");
    if (saved_len[i_cc] != 2 * sd || saved_len[i_ap] != seq || saved_len[i_a] != seq ||
        (i_tp >= 0 && (saved_len[i_tp] != seq || saved_len[i_t] != seq)) ||
        (i_e >= 0 && saved_len[i_e] != seq) || (i_s >= 0 && saved_len[i_s] != tr) ||
        (i_kn >= 0 && (saved_len[i_kn] != seq || saved_len[i_kn + 1] != seq)))
        return orl_fail(NLH_ERR_INVALID_ARG, "rule adapter: a cache buffer has the wrong length");
    if (d > 1024) return orl_fail(NLH_ERR_UNSUPPORTED, "rule adapter: d > 1024");

    cudaStream_t st = current_stream();
    Staging sg;
    float* flat = sg.upload(saved[1], nflat, st);
    float* emb = sg.upload(saved[2], sd, st);
    float* ms = sg.upload(saved[base], tr, st);
    float* ss = (i_s >= 0) ? sg.upload(saved[i_s], tr, st) : nullptr;
    float* k = sg.upload(saved[i_k], sd, st);
    float* v = sg.upload(saved[i_k + 1], sd, st);
    float* q = sg.upload(saved[i_k + 2], sd, st);
    float* cc = sg.upload(saved[i_cc], 2 * sd, st);
    float* ap = sg.upload(saved[i_ap], seq, st);
    float* al = sg.upload(saved[i_a], seq, st);
    float* tp = (i_tp >= 0) ? sg.upload(saved[i_tp], seq, st) : nullptr;
    float* th = (i_t >= 0) ? sg.upload(saved[i_t], seq, st) : nullptr;
    float* et = (i_e >= 0) ? sg.upload(saved[i_e], seq, st) : nullptr;
    float* kn = (i_kn >= 0) ? sg.upload(saved[i_kn], seq, st) : nullptr;
    float* qn = (i_kn >= 0) ? sg.upload(saved[i_kn + 1], seq, st) : nullptr;
    float* dy = sg.upload(d_outputs[0], sd, st);
    float *gk = sg.zeros(sd, st), *gv = sg.zeros(sd, st), *gq = sg.zeros(sd, st);
    float *ga = sg.zeros(seq, st), *gt = sg.zeros(seq, st), *ge = sg.zeros(seq, st);
    float *gm = sg.zeros(dd, st), *gs = sg.zeros(dd, st);
    float* d_kvq = sg.empty(3 * sd);
    float* dpre = sg.empty(3 * seq);
    float* w16 = sg.empty(3 * dd);
    float* d_flat = sg.zeros(in_len[1], st);
    float* d_emb = sg.empty(sd);
    if (!sg.ok) return orl_fail(NLH_ERR_CUDA, "rule adapter: device staging failed");

    // (1) inner-loop backward on the saved trajectory
    nlh_clear_status();
    const int S = (int)seq, D = (int)d;
    if (rule == 0) delta_backward_f32_cuda(k, v, q, al, th, ms, dy, gk, gv, gq, ga, gt, gm, S, D, 1, 0.0f);
    else if (rule == 1) titans_backward_f32_cuda(k, v, q, al, th, et, ms, ss, dy, gk, gv, gq, ga, gt, ge, gm, gs, S, D, 1, 0.0f);
    else hebbian_backward_f32_cuda(k, v, q, al, ms, dy, gk, gv, gq, ga, gm, S, D);
    if (nlh_last_status() != NLH_OK) return nlh_last_status();

    // (2) gate adjoints, gate -> k/v gradient, L2-normalisation Jacobian
    GateArgs g;
    g.k = k; g.v = v; g.q = q; g.dk = gk; g.dv = gv; g.dq = gq;
    g.d_alpha = ga; g.d_theta = gt; g.d_eta = ge;
    g.alpha_pre = ap; g.alpha = al; g.theta_pre = tp; g.theta = th; g.eta = et;
    g.w_alpha = flat + 3 * dd; g.w_theta = flat + 3 * dd + (2 * d + 1); g.w_eta = flat + 3 * dd + 2 * (2 * d + 1);
    g.k_norm = kn; g.q_norm = qn; g.d_kvq = d_kvq; g.dpre = dpre;
    g.a_lo = a_lo; g.a_hi = a_hi; g.t_lo = t_lo; g.t_hi = t_hi;
    g.s = S; g.d = D; g.rule = rule;
    rule_gate_bwd_kernel<<<S, 128, 0, st>>>(g);
    // (3) gate weight gradients straight into the flat gradient
    rule_gate_wgrad_kernel<<<(3 * (2 * D + 1) + 127) / 128, 128, 0, st>>>(dpre, cc, d_flat, S, D, 3 * dd);
    // (4) projection backward
    bf16_round_kernel<<<(unsigned)((3 * dd + 255) / 256 < 2048 ? (3 * dd + 255) / 256 : 2048), 256, 0, st>>>(flat, w16, 3 * dd);
    {
        dim3 gw((unsigned)((d + 31) / 32), (unsigned)((3 * d + 31) / 32));
        // d[W_k; W_v; W_q] [3d, d] = d_kvq^T [3d, s] embedded [s, d]
        orl_sgemm_kernel<true><<<gw, 256, 0, st>>>(d_kvq, 3 * D, emb, D, d_flat, D, 3 * D, D, S);
        dim3 ge2((unsigned)((d + 31) / 32), (unsigned)((seq + 31) / 32));
        // d_embedded [s, d] = d_kvq [s, 3d] [W_k; W_v; W_q] [3d, d]
        orl_sgemm_kernel<false><<<ge2, 256, 0, st>>>(d_kvq, 3 * D, w16, D, d_emb, D, S, D, 3 * D);
    }
    if (!check_launch("nlh_opaque_backward")) return NLH_ERR_CUDA;
    if (!download(d_inputs[0], d_emb, sd, st) || !download(d_inputs[1], d_flat, in_len[1], st))
        return orl_fail(NLH_ERR_CUDA, "rule adapter: download failed");
    if (cudaStreamSynchronize(st) != cudaSuccess) return orl_fail(NLH_ERR_CUDA, "stream synchronisation failed");
    (void)n_out;
    return NLH_OK;
}

}  // namespace nlh
