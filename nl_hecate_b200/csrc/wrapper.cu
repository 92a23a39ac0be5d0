// Fused rule-wrapper and MAG-block glue around the memory kernels.
//
// level_prep   : from the projected [tokens, 3*d_model] (k | v | q) rows to what the
//                per-head recurrence consumes: L2-normalised k,q, raw v in [B*H, s, hd]
//                layout, and the three gates broadcast to heads — one kernel instead of
//                the reference's l2_normalize_rows x2, gate_compute x3, clamp,
//                transpose_heads x3, broadcast_gates x3 (core/src/gpu_forward.rs:1339-1382).
//                Backward twin: gate activation backward, gate->k/v gradient, gate weight
//                gradients, L2-norm backward, inverse head transpose
//                (core/src/gpu_backward.rs:2047-2115, gate_backward.cu, l2_normalize.cu).
// mag_combine  : out = x + attn_proj * sigmoid(sum_l w_l * upsample(y_l)) reading the
//                per-head level outputs directly (core/src/gpu_stacked_forward.rs:1935-1960),
//                and its backward.
// Gate activations saturate at |x| >= 15 like core/src/tensor.rs:199-227.
#include <cuda_bf16.h>

#include "nlh_common.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {

constexpr int WR_THREADS = 128;
constexpr int WR_TOK_PER_CTA = 32;     // most tokens per CTA in level_prep backward
constexpr int WR_MAX_LEVELS = 4;

__device__ __forceinline__ float wr_sigmoid(float x)
{
    if (x >= 15.0f) return 1.0f;
    if (x <= -15.0f) return 0.0f;
    return 1.0f / (1.0f + expf(-x));
}
__device__ __forceinline__ float wr_softplus(float x)
{
    if (x >= 15.0f) return x;
    if (x <= -15.0f) return 0.0f;
    return logf(1.0f + expf(x));
}
__device__ __forceinline__ float ld_as_float(const float* p) { return *p; }
__device__ __forceinline__ float ld_as_float(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_from_float(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_from_float(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// Sum NV values over the CTA; result broadcast to every thread. red: NV * 32 floats.
template <int NV>
__device__ __forceinline__ void block_sum_n(float (&v)[NV], float* red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        v[i] = warp_sum(v[i]);
        if (lane == 0) red[i * 32 + warp] = v[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NV; i++) {
        float t = 0.0f;
        for (int w = 0; w < nw; w++) t += red[i * 32 + w];
        v[i] = t;
    }
    __syncthreads();
}

// ───────────────────────── level prep forward ─────────────────────────────
// One CTA per token. kvq row = [k(d) | v(d) | q(d)].
template <typename TIN>
__global__ void __launch_bounds__(WR_THREADS) level_prep_fwd_kernel(
    const TIN* __restrict__ kvq, const float* __restrict__ w_gates, const float* __restrict__ b_alpha,
    const float* __restrict__ b_theta, const float* __restrict__ b_eta,
    float* __restrict__ k_ph, float* __restrict__ v_ph, float* __restrict__ q_ph,
    float* __restrict__ alpha_ph, float* __restrict__ theta_ph, float* __restrict__ eta_ph,
    float* __restrict__ k_norm, float* __restrict__ q_norm, int sf, int d, int H)
{
    extern __shared__ float sm[];
    float* ks = sm; float* vs = sm + d; float* qs = sm + 2 * d; float* red = sm + 3 * d;  // [8*32]
    const int tok = blockIdx.x, b = tok / sf, t = tok - b * sf;
    const int hd = d / H;
    const TIN* row = kvq + (size_t)tok * 3 * d;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float kj = ld_as_float(row + j), vj = ld_as_float(row + d + j), qj = ld_as_float(row + 2 * d + j);
        ks[j] = kj; vs[j] = vj; qs[j] = qj;
        acc[0] += kj * kj; acc[1] += qj * qj;
#pragma unroll
        for (int g = 0; g < 3; g++) {
            acc[2 + g] += kj * w_gates[(size_t)g * 2 * d + j];
            acc[5 + g] += vj * w_gates[(size_t)g * 2 * d + d + j];
        }
    }
    block_sum_n<8>(acc, red);
    const float kn = sqrtf(acc[0]), qn = sqrtf(acc[1]);
    const float ki = 1.0f / fmaxf(kn, 1e-8f), qi = 1.0f / fmaxf(qn, 1e-8f);
    const float al = wr_sigmoid(acc[2] * ki + acc[5] + *b_alpha);
    const float th = wr_softplus(acc[3] * ki + acc[6] + *b_theta);
    const float et = wr_sigmoid(acc[4] * ki + acc[7] + *b_eta);
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const int h = j / hd, w = j - h * hd;
        const size_t dst = (((size_t)b * H + h) * sf + t) * hd + w;
        k_ph[dst] = ks[j] * ki; v_ph[dst] = vs[j]; q_ph[dst] = qs[j] * qi;
    }
    if (threadIdx.x < H) {
        const size_t g = ((size_t)b * H + threadIdx.x) * sf + t;
        alpha_ph[g] = al; theta_ph[g] = th; eta_ph[g] = et;
    }
    if (threadIdx.x == 0) { k_norm[tok] = kn; q_norm[tok] = qn; }
}

// Warp-per-token variant for d % 8 == 0, head_dim % 8 == 0, d <= 1024: lane owns the 8-element
// chunks c = lane + 32*i (i < NC) of each of k, v, q in registers, so the token is read once with
// 16-byte loads, reduced with shuffles only (no barrier), and written with 16-byte stores.
__device__ __forceinline__ void ld8(const float* p, float (&x)[8])
{
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&x)[8])
{
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        x[2 * i] = f.x; x[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void st8(float* p, const float (&x)[8], float s)
{
    *reinterpret_cast<float4*>(p) = make_float4(x[0] * s, x[1] * s, x[2] * s, x[3] * s);
    *reinterpret_cast<float4*>(p + 4) = make_float4(x[4] * s, x[5] * s, x[6] * s, x[7] * s);
}

constexpr int LPW_WARPS = 4;

template <typename TIN, int NC>
__global__ void __launch_bounds__(LPW_WARPS * 32) level_prep_fwd_warp_kernel(
    const TIN* __restrict__ kvq, const float* __restrict__ w_gates, const float* __restrict__ b_alpha,
    const float* __restrict__ b_theta, const float* __restrict__ b_eta,
    float* __restrict__ k_ph, float* __restrict__ v_ph, float* __restrict__ q_ph,
    float* __restrict__ alpha_ph, float* __restrict__ theta_ph, float* __restrict__ eta_ph,
    float* __restrict__ k_norm, float* __restrict__ q_norm, int n_tok, int sf, int d, int H)
{
    const int lane = threadIdx.x & 31;
    const int tok = blockIdx.x * LPW_WARPS + (threadIdx.x >> 5);
    if (tok >= n_tok) return;
    const int b = tok / sf, t = tok - b * sf;
    const int hd = d / H, nc = d >> 3;
    const TIN* row = kvq + (size_t)tok * 3 * d;
    float kk[NC][8], vv[NC][8], qq[NC][8];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NC; i++) {
        const int c = lane + 32 * i;
        if (c < nc) {
            ld8(row + 8 * c, kk[i]); ld8(row + d + 8 * c, vv[i]); ld8(row + 2 * d + 8 * c, qq[i]);
            float wk[3][8], wv[3][8];
#pragma unroll
            for (int g = 0; g < 3; g++) {
                ld8(w_gates + (size_t)g * 2 * d + 8 * c, wk[g]);
                ld8(w_gates + (size_t)g * 2 * d + d + 8 * c, wv[g]);
            }
#pragma unroll
            for (int e = 0; e < 8; e++) {
                acc[0] += kk[i][e] * kk[i][e]; acc[1] += qq[i][e] * qq[i][e];
#pragma unroll
                for (int g = 0; g < 3; g++) { acc[2 + g] += kk[i][e] * wk[g][e]; acc[5 + g] += vv[i][e] * wv[g][e]; }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < 8; a++) acc[a] = warp_sum(acc[a]);
    const float kn = sqrtf(acc[0]), qn = sqrtf(acc[1]);
    const float ki = 1.0f / fmaxf(kn, 1e-8f), qi = 1.0f / fmaxf(qn, 1e-8f);
#pragma unroll
    for (int i = 0; i < NC; i++) {
        const int c = lane + 32 * i;
        if (c < nc) {
            const int j = 8 * c, h = j / hd, w = j - h * hd;
            const size_t dst = (((size_t)b * H + h) * sf + t) * hd + w;
            st8(k_ph + dst, kk[i], ki); st8(v_ph + dst, vv[i], 1.0f); st8(q_ph + dst, qq[i], qi);
        }
    }
    if (lane < H) {
        const size_t g = ((size_t)b * H + lane) * sf + t;
        alpha_ph[g] = wr_sigmoid(acc[2] * ki + acc[5] + *b_alpha);
        theta_ph[g] = wr_softplus(acc[3] * ki + acc[6] + *b_theta);
        eta_ph[g] = wr_sigmoid(acc[4] * ki + acc[7] + *b_eta);
    }
    if (lane == 0) { k_norm[tok] = kn; q_norm[tok] = qn; }
}

// ───────────────────────── level prep backward ────────────────────────────
// One CTA per tok_per_cta tokens (see lp_tok_per_cta); thread owns elements j = tid + i*WR_THREADS (i < NE) of
// each d-vector, so the gate-weight gradient accumulates in registers across the CTA's tokens
// and is written once as a per-CTA partial [n_cta, 3, 2d] (summed by the caller).
template <typename TIN, int NE>
__global__ void __launch_bounds__(WR_THREADS) level_prep_bwd_kernel(
    const float* __restrict__ k_ph, const float* __restrict__ v_ph, const float* __restrict__ q_ph,
    const float* __restrict__ alpha_ph, const float* __restrict__ theta_ph, const float* __restrict__ eta_ph,
    const float* __restrict__ k_norm, const float* __restrict__ q_norm,
    const float* __restrict__ dk_ph, const float* __restrict__ dv_ph, const float* __restrict__ dq_ph,
    const float* __restrict__ dalpha_ph, const float* __restrict__ dtheta_ph, const float* __restrict__ deta_ph,
    const float* __restrict__ w_gates, TIN* __restrict__ d_kvq, float* __restrict__ dw_partial,
    float* __restrict__ db_partial, int n_tok, int sf, int d, int H, int tok_per_cta)
{
    __shared__ float red[5 * 32];
    const int hd = d / H;
    float dwk[3][NE], dwv[3][NE], db[3] = {0.f, 0.f, 0.f};
#pragma unroll
    for (int g = 0; g < 3; g++)
#pragma unroll
        for (int i = 0; i < NE; i++) { dwk[g][i] = 0.f; dwv[g][i] = 0.f; }
    const int tok0 = blockIdx.x * tok_per_cta;
    const int tok1 = min(tok0 + tok_per_cta, n_tok);
    for (int tok = tok0; tok < tok1; tok++) {
        const int b = tok / sf, t = tok - b * sf;
        const size_t g0 = ((size_t)b * H) * sf + t;       // head 0 gate slot; heads are sf apart
        const float al = alpha_ph[g0], th = theta_ph[g0], et = eta_ph[g0];
        float kh[NE], vv[NE], qh[NE], gk[NE], gv[NE], gq[NE];
        float s[5] = {0.f, 0.f, 0.f, 0.f, 0.f};   // d_alpha, d_theta, d_eta (head sums), dk.k, dq.q
        if (threadIdx.x < H) {
            const size_t gi = g0 + (size_t)threadIdx.x * sf;
            s[0] = dalpha_ph[gi]; s[1] = dtheta_ph[gi]; s[2] = deta_ph[gi];
        }
#pragma unroll
        for (int i = 0; i < NE; i++) {
            const int j = threadIdx.x + i * WR_THREADS;
            if (j < d) {
                const int h = j / hd, w = j - h * hd;
                const size_t src = (((size_t)b * H + h) * sf + t) * hd + w;
                kh[i] = k_ph[src]; vv[i] = v_ph[src]; qh[i] = q_ph[src];
                gk[i] = dk_ph[src]; gv[i] = dv_ph[src]; gq[i] = dq_ph[src];
            } else { kh[i] = vv[i] = qh[i] = gk[i] = gv[i] = gq[i] = 0.f; }
        }
        // gate head sums first (the gate -> k gradient enters the k.dk dot product)
        {
            float hs[3] = {s[0], s[1], s[2]};
            block_sum_n<3>(hs, red);
            s[0] = hs[0]; s[1] = hs[1]; s[2] = hs[2];
        }
        const float dpre[3] = {s[0] * al * (1.0f - al), s[1] * (1.0f - expf(-th)), s[2] * et * (1.0f - et)};
        float dots[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < NE; i++) {
            const int j = threadIdx.x + i * WR_THREADS;
            if (j < d) {
#pragma unroll
                for (int g = 0; g < 3; g++) {
                    gk[i] += dpre[g] * w_gates[(size_t)g * 2 * d + j];
                    gv[i] += dpre[g] * w_gates[(size_t)g * 2 * d + d + j];
                    dwk[g][i] += dpre[g] * kh[i];
                    dwv[g][i] += dpre[g] * vv[i];
                }
                dots[0] += gk[i] * kh[i];
                dots[1] += gq[i] * qh[i];
            }
        }
        if (threadIdx.x == 0) { db[0] += dpre[0]; db[1] += dpre[1]; db[2] += dpre[2]; }
        block_sum_n<2>(dots, red);
        const float kn = k_norm[tok], qn = q_norm[tok];
        TIN* orow = d_kvq + (size_t)tok * 3 * d;
#pragma unroll
        for (int i = 0; i < NE; i++) {
            const int j = threadIdx.x + i * WR_THREADS;
            if (j < d) {
                // sphere Jacobian of x/||x|| (core/src/tensor.rs:320-351)
                const float dk = (kn >= 1e-8f) ? (gk[i] - kh[i] * dots[0]) / kn : gk[i] * 1e8f;
                const float dq = (qn >= 1e-8f) ? (gq[i] - qh[i] * dots[1]) / qn : gq[i] * 1e8f;
                st_from_float(orow + j, dk);
                st_from_float(orow + d + j, gv[i]);
                st_from_float(orow + 2 * d + j, dq);
            }
        }
    }
    float* dwp = dw_partial + (size_t)blockIdx.x * 3 * 2 * d;
#pragma unroll
    for (int g = 0; g < 3; g++)
#pragma unroll
        for (int i = 0; i < NE; i++) {
            const int j = threadIdx.x + i * WR_THREADS;
            if (j < d) { dwp[(size_t)g * 2 * d + j] = dwk[g][i]; dwp[(size_t)g * 2 * d + d + j] = dwv[g][i]; }
        }
    if (threadIdx.x == 0) {
        db_partial[blockIdx.x * 3 + 0] = db[0];
        db_partial[blockIdx.x * 3 + 1] = db[1];
        db_partial[blockIdx.x * 3 + 2] = db[2];
    }
}


// Warp-per-token backward (same conditions as level_prep_fwd_warp_kernel): writes d_kvq and the
// gate pre-activation gradients dpre [tokens, 3] (alpha, theta, eta); the gate-weight gradient,
// a reduction over tokens, is left to gate_wgrad_kernel so that this kernel stays light.
__device__ __forceinline__ void st8_as(float* p, const float (&x)[8]) { st8(p, x, 1.0f); }
__device__ __forceinline__ void st8_as(__nv_bfloat16* p, const float (&x)[8])
{
    uint4 u;
    __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(x[4], x[5]), e = __floats2bfloat162_rn(x[6], x[7]);
    u.x = *reinterpret_cast<unsigned*>(&a); u.y = *reinterpret_cast<unsigned*>(&b);
    u.z = *reinterpret_cast<unsigned*>(&c); u.w = *reinterpret_cast<unsigned*>(&e);
    *reinterpret_cast<uint4*>(p) = u;
}

template <typename TIN, int NC>
__global__ void __launch_bounds__(LPW_WARPS * 32) level_prep_bwd_warp_kernel(
    const float* __restrict__ k_ph, const float* __restrict__ v_ph, const float* __restrict__ q_ph,
    const float* __restrict__ alpha_ph, const float* __restrict__ theta_ph, const float* __restrict__ eta_ph,
    const float* __restrict__ k_norm, const float* __restrict__ q_norm,
    const float* __restrict__ dk_ph, const float* __restrict__ dv_ph, const float* __restrict__ dq_ph,
    const float* __restrict__ dalpha_ph, const float* __restrict__ dtheta_ph, const float* __restrict__ deta_ph,
    const float* __restrict__ w_gates, TIN* __restrict__ d_kvq, float* __restrict__ dpre_out,
    int n_tok, int sf, int d, int H)
{
    const int lane = threadIdx.x & 31;
    const int tok = blockIdx.x * LPW_WARPS + (threadIdx.x >> 5);
    if (tok >= n_tok) return;
    const int hd = d / H, nc = d >> 3;
    const int b = tok / sf, t = tok - b * sf;
    const size_t g0 = ((size_t)b * H) * sf + t;       // head 0 gate slot; heads are sf apart
    const float al = alpha_ph[g0], th = theta_ph[g0], et = eta_ph[g0];
    const float kn = k_norm[tok], qn = q_norm[tok];
    float s0 = 0.f, s1 = 0.f, s2 = 0.f;
    if (lane < H) {
        const size_t gi = g0 + (size_t)lane * sf;
        s0 = dalpha_ph[gi]; s1 = dtheta_ph[gi]; s2 = deta_ph[gi];
    }
    float kh[NC][8], qh[NC][8], gk[NC][8], gq[NC][8], gv[NC][8];
#pragma unroll
    for (int i = 0; i < NC; i++) {
        const int c = lane + 32 * i;
        if (c < nc) {
            const int j = 8 * c, h = j / hd, w = j - h * hd;
            const size_t src = (((size_t)b * H + h) * sf + t) * hd + w;
            ld8(k_ph + src, kh[i]); ld8(q_ph + src, qh[i]);
            ld8(dk_ph + src, gk[i]); ld8(dv_ph + src, gv[i]); ld8(dq_ph + src, gq[i]);
        }
    }
    s0 = warp_sum(s0); s1 = warp_sum(s1); s2 = warp_sum(s2);
    const float dpre[3] = {s0 * al * (1.0f - al), s1 * (1.0f - expf(-th)), s2 * et * (1.0f - et)};
    if (lane < 3) dpre_out[(size_t)tok * 3 + lane] = lane == 0 ? dpre[0] : lane == 1 ? dpre[1] : dpre[2];
    float dot_k = 0.f, dot_q = 0.f;
    TIN* orow = d_kvq + (size_t)tok * 3 * d;
#pragma unroll
    for (int i = 0; i < NC; i++) {
        const int c = lane + 32 * i;
        if (c < nc) {
            const int j = 8 * c;
#pragma unroll
            for (int g = 0; g < 3; g++) {
                float wk[8], wv[8];
                ld8(w_gates + (size_t)g * 2 * d + j, wk);
                ld8(w_gates + (size_t)g * 2 * d + d + j, wv);
#pragma unroll
                for (int e = 0; e < 8; e++) { gk[i][e] += dpre[g] * wk[e]; gv[i][e] += dpre[g] * wv[e]; }
            }
#pragma unroll
            for (int e = 0; e < 8; e++) { dot_k += gk[i][e] * kh[i][e]; dot_q += gq[i][e] * qh[i][e]; }
            st8_as(orow + d + j, gv[i]);
        }
    }
    dot_k = warp_sum(dot_k);
    dot_q = warp_sum(dot_q);
    const float kinv = (kn >= 1e-8f) ? 1.0f / kn : 1e8f, qinv = (qn >= 1e-8f) ? 1.0f / qn : 1e8f;
    const float kd = (kn >= 1e-8f) ? dot_k : 0.f, qd = (qn >= 1e-8f) ? dot_q : 0.f;
#pragma unroll
    for (int i = 0; i < NC; i++) {
        const int c = lane + 32 * i;
        if (c < nc) {
            // sphere Jacobian of x/||x|| (core/src/tensor.rs:320-351)
            float ok[8], oq[8];
#pragma unroll
            for (int e = 0; e < 8; e++) {
                ok[e] = (gk[i][e] - kh[i][e] * kd) * kinv;
                oq[e] = (gq[i][e] - qh[i][e] * qd) * qinv;
            }
            st8_as(orow + 8 * c, ok);
            st8_as(orow + 2 * d + 8 * c, oq);
        }
    }
}

// Gate-weight and gate-bias gradients: dw[g, :] = sum_tok dpre[tok, g] * [k_hat(tok) | v(tok)],
// db[g] = sum_tok dpre[tok, g]. One CTA per tok_per_cta consecutive tokens writes one partial
// row [3, 2d] (+ [3]); the caller sums the rows. Thread owns 4 consecutive columns of k and of v
// per pass (d <= 4 * blockDim.x * WG_PASSES).
constexpr int WG_THREADS = 128;
constexpr int WG_PASSES = 2;      // d_model <= 1024
__global__ void __launch_bounds__(WG_THREADS) gate_wgrad_kernel(
    const float* __restrict__ dpre, const float* __restrict__ k_ph, const float* __restrict__ v_ph,
    float* __restrict__ dw_partial, float* __restrict__ db_partial, int n_tok, int sf, int d, int H,
    int tok_per_cta)
{
    const int hd = d / H;
    const int tok0 = blockIdx.x * tok_per_cta;
    const int tok1 = min(tok0 + tok_per_cta, n_tok);
    float4 ak[WG_PASSES][3], av[WG_PASSES][3];
#pragma unroll
    for (int p = 0; p < WG_PASSES; p++)
#pragma unroll
        for (int g = 0; g < 3; g++) { ak[p][g] = make_float4(0.f, 0.f, 0.f, 0.f); av[p][g] = make_float4(0.f, 0.f, 0.f, 0.f); }
    float db[3] = {0.f, 0.f, 0.f};
    for (int tok = tok0; tok < tok1; tok++) {
        const int b = tok / sf, t = tok - b * sf;
        const float p0 = dpre[(size_t)tok * 3], p1 = dpre[(size_t)tok * 3 + 1], p2 = dpre[(size_t)tok * 3 + 2];
        db[0] += p0; db[1] += p1; db[2] += p2;
#pragma unroll
        for (int p = 0; p < WG_PASSES; p++) {
            const int j = 4 * (threadIdx.x + p * WG_THREADS);
            if (j < d) {
                const int h = j / hd, w = j - h * hd;
                const size_t src = (((size_t)b * H + h) * sf + t) * hd + w;
                const float4 kv = *reinterpret_cast<const float4*>(k_ph + src);
                const float4 vv = *reinterpret_cast<const float4*>(v_ph + src);
                ak[p][0].x += p0 * kv.x; ak[p][0].y += p0 * kv.y; ak[p][0].z += p0 * kv.z; ak[p][0].w += p0 * kv.w;
                ak[p][1].x += p1 * kv.x; ak[p][1].y += p1 * kv.y; ak[p][1].z += p1 * kv.z; ak[p][1].w += p1 * kv.w;
                ak[p][2].x += p2 * kv.x; ak[p][2].y += p2 * kv.y; ak[p][2].z += p2 * kv.z; ak[p][2].w += p2 * kv.w;
                av[p][0].x += p0 * vv.x; av[p][0].y += p0 * vv.y; av[p][0].z += p0 * vv.z; av[p][0].w += p0 * vv.w;
                av[p][1].x += p1 * vv.x; av[p][1].y += p1 * vv.y; av[p][1].z += p1 * vv.z; av[p][1].w += p1 * vv.w;
                av[p][2].x += p2 * vv.x; av[p][2].y += p2 * vv.y; av[p][2].z += p2 * vv.z; av[p][2].w += p2 * vv.w;
            }
        }
    }
    float* dwp = dw_partial + (size_t)blockIdx.x * 3 * 2 * d;
#pragma unroll
    for (int p = 0; p < WG_PASSES; p++) {
        const int j = 4 * (threadIdx.x + p * WG_THREADS);
        if (j < d) {
#pragma unroll
            for (int g = 0; g < 3; g++) {
                *reinterpret_cast<float4*>(dwp + (size_t)g * 2 * d + j) = ak[p][g];
                *reinterpret_cast<float4*>(dwp + (size_t)g * 2 * d + d + j) = av[p][g];
            }
        }
    }
    if (threadIdx.x == 0) {
        db_partial[blockIdx.x * 3 + 0] = db[0];
        db_partial[blockIdx.x * 3 + 1] = db[1];
        db_partial[blockIdx.x * 3 + 2] = db[2];
    }
}

// ───────────────────────── MAG combine ────────────────────────────────────
struct CombineLevels {
    const float* y[WR_MAX_LEVELS];   // per-head level outputs [B*H, S/c, hd]
    int c[WR_MAX_LEVELS];            // pooling factor of the level (tokens per level token)
    FastDiv cdiv[WR_MAX_LEVELS];     // division by c[l]
    FastDiv sdiv;                    // division by the sequence length
    int k;
};

// Gate of the MAG combine: sigmoid with the fast exponential and reciprocal (relative error about
// 1e-6 over the unsaturated range; saturates like wr_sigmoid).
__device__ __forceinline__ float combine_sigmoid(float x)
{
    if (x >= 15.0f) return 1.0f;
    if (x <= -15.0f) return 0.0f;
    return __fdividef(1.0f, 1.0f + __expf(-x));
}

template <typename TIN>
__device__ __forceinline__ float4 ld4(const TIN* p);
template <>
__device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p)
{
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v)
{
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<unsigned*>(&a); r.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

// Element-wise passes over [rows, d] walk whole rows: a thread keeps one float4 column chunk
// and steps over rows, so the per-element index arithmetic is one 32-bit division per row
// instead of 64-bit divisions per element. Needs d/4 <= blockDim.x.
struct RowWalk {
    int c4;      // float4 column chunk of this thread
    int row;     // first row (INT_MAX for threads beyond the last whole row of the CTA)
    int step;    // rows between passes
};
__device__ __forceinline__ RowWalk row_walk(int d4)
{
    const int rpc = blockDim.x / d4;
    const int r = threadIdx.x / d4;
    RowWalk w;
    w.c4 = threadIdx.x - r * d4;
    w.row = (r < rpc) ? blockIdx.x * rpc + r : 0x7fffffff;
    w.step = gridDim.x * rpc;
    return w;
}

// Warp per row of [B*S, d]: lane owns the float4 chunks c = lane + 32 i (i < NV) of the row, so the
// row -> (sequence, token, level token) index arithmetic is done once per row instead of once per
// element, the per-chunk head offsets are fixed for the whole kernel, and a lane has NV
// independent load groups in flight.
constexpr int CMB_WARPS = 8;

struct CombineRow {
    size_t base[WR_MAX_LEVELS];     // element offset of (sequence b, level token of t, head 0, 0) in y_l
};
__device__ __forceinline__ CombineRow combine_row(const CombineLevels& L, int row, int S, int H, int hd)
{
    CombineRow r;
    const int b = fd_div(row, L.sdiv), t = row - b * S;
#pragma unroll
    for (int l = 0; l < WR_MAX_LEVELS; l++) {
        const int sfl = fd_div(S, L.cdiv[l]);
        r.base[l] = ((size_t)b * H * sfl + fd_div(t, L.cdiv[l])) * hd;
    }
    return r;
}

// out = x + attn_proj * sigmoid(y_comb)
template <typename TIN, int NV>
__global__ void __launch_bounds__(CMB_WARPS * 32) mag_combine_fwd_kernel(
    const float* __restrict__ x, const TIN* __restrict__ attn_proj, const float* __restrict__ wts,
    CombineLevels L, float* __restrict__ out, int B, int S, int d, int H)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hd = d / H, nv = d >> 2, n_rows = B * S;
    float wl[WR_MAX_LEVELS];
    int hstride[WR_MAX_LEVELS];                 // elements between heads in y_l
#pragma unroll
    for (int l = 0; l < WR_MAX_LEVELS; l++) {
        wl[l] = l < L.k ? wts[l] : 0.f;
        hstride[l] = fd_div(S, L.cdiv[l]) * hd;
    }
    int hh[NV], ww[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) { const int j = 4 * (lane + 32 * i); hh[i] = j / hd; ww[i] = j - hh[i] * hd; }
    for (int row = blockIdx.x * CMB_WARPS + warp; row < n_rows; row += gridDim.x * CMB_WARPS) {
        const CombineRow R = combine_row(L, row, S, H, hd);
        const size_t ro = (size_t)row * d;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int c = lane + 32 * i;
            if (c < nv) {
                float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int l = 0; l < WR_MAX_LEVELS; l++)
                    if (l < L.k) {
                        const float4 v = *reinterpret_cast<const float4*>(L.y[l] + R.base[l] + (size_t)hh[i] * hstride[l] + ww[i]);
                        y.x += wl[l] * v.x; y.y += wl[l] * v.y; y.z += wl[l] * v.z; y.w += wl[l] * v.w;
                    }
                const float4 xa = ld4<float>(x + ro + 4 * c), ap = ld4<TIN>(attn_proj + ro + 4 * c);
                float4 o;
                o.x = xa.x + ap.x * combine_sigmoid(y.x); o.y = xa.y + ap.y * combine_sigmoid(y.y);
                o.z = xa.z + ap.z * combine_sigmoid(y.z); o.w = xa.w + ap.w * combine_sigmoid(y.w);
                st4(out + ro + 4 * c, o);
            }
        }
    }
}

// Optional per-level outputs of the combine backward: for a level with pool factor 1,
// dy[l] [B*H, S, hd] receives w_l * d_ycomb in the per-head layout (NULL = not wanted).
struct CombineGrads {
    float* dy[WR_MAX_LEVELS];
};

// d_attn_proj = d_out * gate ; d_ycomb = d_out * attn_proj * gate * (1 - gate) ;
// dw_partial[cta][l] = sum d_ycomb * upsample(y_l)   (gradient of the level weights)
template <typename TIN, int NV>
__global__ void __launch_bounds__(CMB_WARPS * 32) mag_combine_bwd_kernel(
    const float* __restrict__ d_out, const TIN* __restrict__ attn_proj, const float* __restrict__ wts,
    CombineLevels L, TIN* __restrict__ d_attn_proj, float* __restrict__ d_ycomb,
    float* __restrict__ dw_partial, CombineGrads G, int B, int S, int d, int H)
{
    __shared__ float red[WR_MAX_LEVELS * 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hd = d / H, nv = d >> 2, n_rows = B * S;
    float dw[WR_MAX_LEVELS] = {0.f, 0.f, 0.f, 0.f};
    float wl[WR_MAX_LEVELS];
    int hstride[WR_MAX_LEVELS];
#pragma unroll
    for (int l = 0; l < WR_MAX_LEVELS; l++) {
        wl[l] = l < L.k ? wts[l] : 0.f;
        hstride[l] = fd_div(S, L.cdiv[l]) * hd;
    }
    int hh[NV], ww[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) { const int j = 4 * (lane + 32 * i); hh[i] = j / hd; ww[i] = j - hh[i] * hd; }
    for (int row = blockIdx.x * CMB_WARPS + warp; row < n_rows; row += gridDim.x * CMB_WARPS) {
        const CombineRow R = combine_row(L, row, S, H, hd);
        const size_t ro = (size_t)row * d;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int c = lane + 32 * i;
            if (c < nv) {
                float4 yl[WR_MAX_LEVELS];
                float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int l = 0; l < WR_MAX_LEVELS; l++)
                    if (l < L.k) {
                        yl[l] = *reinterpret_cast<const float4*>(L.y[l] + R.base[l] + (size_t)hh[i] * hstride[l] + ww[i]);
                        y.x += wl[l] * yl[l].x; y.y += wl[l] * yl[l].y; y.z += wl[l] * yl[l].z; y.w += wl[l] * yl[l].w;
                    }
                const float4 go = ld4<float>(d_out + ro + 4 * c), ap = ld4<TIN>(attn_proj + ro + 4 * c);
                float4 g, dap, dy;
                g.x = combine_sigmoid(y.x); g.y = combine_sigmoid(y.y); g.z = combine_sigmoid(y.z); g.w = combine_sigmoid(y.w);
                dap.x = go.x * g.x; dap.y = go.y * g.y; dap.z = go.z * g.z; dap.w = go.w * g.w;
                dy.x = go.x * ap.x * g.x * (1.f - g.x); dy.y = go.y * ap.y * g.y * (1.f - g.y);
                dy.z = go.z * ap.z * g.z * (1.f - g.z); dy.w = go.w * ap.w * g.w * (1.f - g.w);
                st4(d_attn_proj + ro + 4 * c, dap);
                st4(d_ycomb + ro + 4 * c, dy);
#pragma unroll
                for (int l = 0; l < WR_MAX_LEVELS; l++) {
                    if (l < L.k) {
                        dw[l] += dy.x * yl[l].x + dy.y * yl[l].y + dy.z * yl[l].z + dy.w * yl[l].w;
                        if (G.dy[l] != nullptr)     // unpooled level (c_l = 1): same layout as y_l, no pooling pass
                            *reinterpret_cast<float4*>(G.dy[l] + R.base[l] + (size_t)hh[i] * hstride[l] + ww[i]) =
                                make_float4(wl[l] * dy.x, wl[l] * dy.y, wl[l] * dy.z, wl[l] * dy.w);
                    }
                }
            }
        }
    }
    block_sum_n<WR_MAX_LEVELS>(dw, red);
    if (threadIdx.x < WR_MAX_LEVELS) dw_partial[blockIdx.x * WR_MAX_LEVELS + threadIdx.x] = dw[threadIdx.x];
}

// dy_ph[(b*H+h), t', w] = scale * sum_{i<c} d_ycomb[b, t'*c + i, h*hd + w]  (adjoint of
// repeat-upsample followed by the level weight), written in the per-head layout.
__global__ void __launch_bounds__(256) pool_to_heads_kernel(
    const float* __restrict__ d_ycomb, const float* __restrict__ wts, int level, int c,
    float* __restrict__ dy_ph, float* __restrict__ sum_out, int B, int S, int d, int H)
{
    const int hd = d / H, d4 = d / 4, sf = S / c;
    const long long n4 = (long long)B * sf * d4;
    const float scale = wts[level];
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const int j = (int)(i % d4) * 4;
        const long long bt = i / d4;
        const int tp = (int)(bt % sf), b = (int)(bt / sf);
        const float* src = d_ycomb + ((size_t)b * S + (size_t)tp * c) * d + j;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < c; q++) {
            const float4 v = *reinterpret_cast<const float4*>(src + (size_t)q * d);
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        const int h = j / hd, w = j - h * hd;
        const size_t o = (((size_t)b * H + h) * sf + tp) * hd + w;
        if (sum_out != nullptr) *reinterpret_cast<float4*>(sum_out + o) = a;
        a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
        *reinterpret_cast<float4*>(dy_ph + o) = a;
    }
}

// Coarser level from a finer level's unscaled sums, both in the per-head layout:
// dy_ph[n, t', :] = scale * sum_{i<f} src[n, t'*f + i, :]  (n = batch*heads rows of hd floats).
__global__ void __launch_bounds__(256) pool_heads_kernel(
    const float* __restrict__ src, const float* __restrict__ wts, int level, int f,
    float* __restrict__ dy_ph, float* __restrict__ sum_out, long long n_out4, int hd4)
{
    const float scale = wts[level];
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_out4;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / hd4;                 // output row (n, t')
        const int w4 = (int)(i - row * hd4);
        const float4* sp = reinterpret_cast<const float4*>(src) + row * f * hd4 + w4;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < f; q++) {
            const float4 v = sp[(size_t)q * hd4];
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        if (sum_out != nullptr) reinterpret_cast<float4*>(sum_out)[i] = a;
        a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
        reinterpret_cast<float4*>(dy_ph)[i] = a;
    }
}

// Mean pooling of token rows for the coarser levels (core/kernels/pool_ops.cu mean_pool_1d):
// out[r, :] = scale * sum_{i<f} src[r*f + i, :], optional unscaled sums for the next level.
template <typename TOUT>
__global__ void __launch_bounds__(256) mean_pool_kernel(const float* __restrict__ src, int f, float scale,
    TOUT* __restrict__ out, float* __restrict__ sum_out, long long n_out4, int d4)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_out4;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / d4;
        const int c4 = (int)(i - row * d4);
        const float4* sp = reinterpret_cast<const float4*>(src) + row * f * d4 + c4;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int q = 0; q < f; q++) {
            const float4 v = sp[(size_t)q * d4];
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        if (sum_out != nullptr) reinterpret_cast<float4*>(sum_out)[i] = a;
        a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
        st4(out + i * 4, a);
    }
}

// Adjoint of the mean pools of up to three levels in one pass:
// out[b, t, :] = sum_l g_l[b, t / c_l, :] / c_l  (core/kernels/pool_ops.cu repeat_upsample_1d + scale).
struct UnpoolSrc {
    const void* g[3];
    int c[3];
    FastDiv cdiv[3];
    FastDiv sdiv;        // division by the sequence length
    int is_bf16[3];
    int n;
};
__global__ void __launch_bounds__(256) unpool_sum_kernel(UnpoolSrc P, float* __restrict__ out,
                                                         long long n4, int S, int d4)
{
    const int n_rows = (int)(n4 / d4);
    const RowWalk rw = row_walk(d4);
    const int c4 = rw.c4;
    for (int r = rw.row; r < n_rows; r += rw.step) {
        const int b = fd_div(r, P.sdiv), t = r - b * S;
        const size_t i = (size_t)r * d4 + c4;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int l = 0; l < 3; l++) {
            if (l < P.n) {
                const long long row = (long long)b * fd_div(S, P.cdiv[l]) + fd_div(t, P.cdiv[l]);
                const size_t o = ((size_t)row * d4 + c4) * 4;
                const float4 v = P.is_bf16[l] ? ld4<__nv_bfloat16>((const __nv_bfloat16*)P.g[l] + o)
                                              : ld4<float>((const float*)P.g[l] + o);
                const float inv = 1.0f / (float)P.c[l];
                a.x += v.x * inv; a.y += v.y * inv; a.z += v.z * inv; a.w += v.w * inv;
            }
        }
        *reinterpret_cast<float4*>(out + i * 4) = a;
    }
}

static int wr_grid(long long items, int per_cta)
{
    long long need = (items + per_cta - 1) / per_cta;
    if (need < 1) need = 1;
    const long long cap = 148LL * 16;
    return (int)(need < cap ? need : cap);
}


// ───────────────────────── partial-row finishers ──────────────────────────
// The backward kernels above leave parameter gradients as per-CTA partial rows. These kernels sum
// the rows and ADD the result into the caller's gradient buffers, so that a training step needs no
// reduction and no accumulation pass of its own.
// Gate weights: thread per column of dw_partial [rows, cols], the rows divided over gridDim.y
// slices (one atomicAdd per column and slice: up to 16 addends per element, in any order); the
// last CTA of slice 0 also sums the three bias columns of db_partial [rows, 3].
__global__ void __launch_bounds__(256) gate_grad_finish_kernel(
    const float* __restrict__ dw_partial, const float* __restrict__ db_partial, int rows_total, int cols,
    float* __restrict__ g_w, float* g_b0, float* g_b1, float* g_b2)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int per = (rows_total + gridDim.y - 1) / gridDim.y;
    const int r_lo = blockIdx.y * per;
    const int rows = min(rows_total, r_lo + per);
    if (c < cols && r_lo < rows) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        int r = r_lo;
        for (; r + 4 <= rows; r += 4) {
            a0 += dw_partial[(size_t)r * cols + c];
            a1 += dw_partial[(size_t)(r + 1) * cols + c];
            a2 += dw_partial[(size_t)(r + 2) * cols + c];
            a3 += dw_partial[(size_t)(r + 3) * cols + c];
        }
        for (; r < rows; r++) a0 += dw_partial[(size_t)r * cols + c];
        const float t = (a0 + a1) + (a2 + a3);
        if (gridDim.y == 1) g_w[c] += t; else atomicAdd(g_w + c, t);
    }
    if (blockIdx.x == gridDim.x - 1 && blockIdx.y == 0 && threadIdx.x < 96) {
        const int g = threadIdx.x >> 5, lane = threadIdx.x & 31;
        float s = 0.f;
        for (int r = lane; r < rows_total; r += 32) s += db_partial[(size_t)r * 3 + g];
        s = warp_sum(s);
        float* dst = g == 0 ? g_b0 : g == 1 ? g_b1 : g_b2;
        if (lane == 0 && dst) dst[0] += s;
    }
}

// Level weights w = softmax(logits): sums dw_partial [rows, WR_MAX_LEVELS] over rows (warp per
// level) and adds the softmax adjoint d_logit_i = w_i (dw_i - sum_j w_j dw_j) into g_logits [k].
__global__ void __launch_bounds__(32 * WR_MAX_LEVELS) level_weight_grad_finish_kernel(
    const float* __restrict__ dw_partial, int rows, int k, const float* __restrict__ weights,
    float* g_logits)
{
    __shared__ float dw[WR_MAX_LEVELS];
    const int g = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float s = 0.f;
    if (g < k)
        for (int r = lane; r < rows; r += 32) s += dw_partial[(size_t)r * WR_MAX_LEVELS + g];
    s = warp_sum(s);
    if (lane == 0) dw[g] = (g < k) ? s : 0.f;
    __syncthreads();
    if (threadIdx.x < k) {
        float dot = 0.f;
        for (int j = 0; j < k; j++) dot += weights[j] * dw[j];
        g_logits[threadIdx.x] += weights[threadIdx.x] * (dw[threadIdx.x] - dot);
    }
}
}  // namespace nlh

using namespace nlh;

static int wr_check(const char* where, int B, int S, int d, int H)
{
    if (B < 0 || S <= 0 || d <= 0 || H <= 0 || d % H != 0 || (d / H) % 4 != 0 || d > 1024 ||
        H > WR_THREADS) {
        record_status(NLH_ERR_INVALID_ARG, where,
                      "need d_model <= 1024, d_model % num_heads == 0, head_dim % 4 == 0");
        return NLH_ERR_INVALID_ARG;
    }
    return NLH_OK;
}

extern "C" {

// Tokens a CTA of the level_prep backward walks through: its per-token block reductions are
// serial, so short inputs (the pooled levels) get fewer tokens per CTA and more CTAs.
static int lp_tok_per_cta(int n_tokens)
{
    int t = (n_tokens + 1023) / 1024;
    return t < 1 ? 1 : (t > WR_TOK_PER_CTA ? WR_TOK_PER_CTA : t);
}

int32_t nlh_level_prep_partial_rows(int32_t n_tokens)
{
    const int t = lp_tok_per_cta(n_tokens);
    return (n_tokens + t - 1) / t;
}

int32_t nlh_level_prep_forward(const void* kvq, int32_t kvq_is_bf16, const float* w_gates,
    const float* b_alpha, const float* b_theta, const float* b_eta, float* k_ph, float* v_ph,
    float* q_ph, float* alpha_ph, float* theta_ph, float* eta_ph, float* k_norm, float* q_norm,
    int32_t batch, int32_t seq, int32_t d_model, int32_t num_heads)
{
    int rc = wr_check("nlh_level_prep_forward", batch, seq, d_model, num_heads);
    if (rc != NLH_OK || batch == 0) return rc;
    const int n_tok = batch * seq;
    const size_t smem = (size_t)(3 * d_model + 8 * 32) * sizeof(float);
    cudaStream_t st = current_stream();
    const bool al16 = ((((uintptr_t)kvq | (uintptr_t)w_gates | (uintptr_t)k_ph | (uintptr_t)v_ph | (uintptr_t)q_ph) & 15) == 0);
    if (d_model % 8 == 0 && (d_model / num_heads) % 8 == 0 && num_heads <= 32 && al16) {
        const int grid = (n_tok + LPW_WARPS - 1) / LPW_WARPS;
        const int ncl = (d_model / 8 + 31) / 32;     // chunks per lane, <= 4 because d_model <= 1024
#define NLH_LP_FWD(T, NC)                                                                         \
    level_prep_fwd_warp_kernel<T, NC><<<grid, LPW_WARPS * 32, 0, st>>>(                              \
        (const T*)kvq, w_gates, b_alpha, b_theta, b_eta, k_ph, v_ph, q_ph, alpha_ph, theta_ph,    \
        eta_ph, k_norm, q_norm, n_tok, seq, d_model, num_heads)
        if (kvq_is_bf16) {
            if (ncl <= 1) NLH_LP_FWD(__nv_bfloat16, 1); else if (ncl <= 2) NLH_LP_FWD(__nv_bfloat16, 2); else NLH_LP_FWD(__nv_bfloat16, 4);
        } else {
            if (ncl <= 1) NLH_LP_FWD(float, 1); else if (ncl <= 2) NLH_LP_FWD(float, 2); else NLH_LP_FWD(float, 4);
        }
#undef NLH_LP_FWD
        return check_launch("nlh_level_prep_forward") ? NLH_OK : NLH_ERR_CUDA;
    }
    if (kvq_is_bf16)
        level_prep_fwd_kernel<__nv_bfloat16><<<n_tok, WR_THREADS, smem, st>>>(
            (const __nv_bfloat16*)kvq, w_gates, b_alpha, b_theta, b_eta, k_ph, v_ph, q_ph, alpha_ph,
            theta_ph, eta_ph, k_norm, q_norm, seq, d_model, num_heads);
    else
        level_prep_fwd_kernel<float><<<n_tok, WR_THREADS, smem, st>>>(
            (const float*)kvq, w_gates, b_alpha, b_theta, b_eta, k_ph, v_ph, q_ph, alpha_ph,
            theta_ph, eta_ph, k_norm, q_norm, seq, d_model, num_heads);
    return check_launch("nlh_level_prep_forward") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_level_prep_backward(const float* k_ph, const float* v_ph, const float* q_ph,
    const float* alpha_ph, const float* theta_ph, const float* eta_ph, const float* k_norm,
    const float* q_norm, const float* dk_ph, const float* dv_ph, const float* dq_ph,
    const float* dalpha_ph, const float* dtheta_ph, const float* deta_ph, const float* w_gates,
    void* d_kvq, int32_t kvq_is_bf16, float* dw_partial, float* db_partial, int32_t batch,
    int32_t seq, int32_t d_model, int32_t num_heads)
{
    int rc = wr_check("nlh_level_prep_backward", batch, seq, d_model, num_heads);
    if (rc != NLH_OK || batch == 0) return rc;
    const int n_tok = batch * seq;
    const int grid = nlh_level_prep_partial_rows(n_tok);
    const int ne = (d_model + WR_THREADS - 1) / WR_THREADS;
    cudaStream_t st = current_stream();
    const bool al16 = ((((uintptr_t)k_ph | (uintptr_t)v_ph | (uintptr_t)q_ph | (uintptr_t)dk_ph | (uintptr_t)dv_ph |
                         (uintptr_t)dq_ph | (uintptr_t)w_gates | (uintptr_t)d_kvq) & 15) == 0);
    if (d_model % 8 == 0 && (d_model / num_heads) % 8 == 0 && num_heads <= 32 && al16 &&
        ((uintptr_t)dw_partial & 15) == 0) {
        float* dpre = (float*)workspace((size_t)n_tok * 3 * sizeof(float));
        if (!dpre) return NLH_ERR_WORKSPACE;
        const int wgrid = (n_tok + LPW_WARPS - 1) / LPW_WARPS;
        const int ncl = (d_model / 8 + 31) / 32;     // chunks per lane, <= 4 because d_model <= 1024
#define NLH_LP_BWDW(T, NC)                                                                       \
    level_prep_bwd_warp_kernel<T, NC><<<wgrid, LPW_WARPS * 32, 0, st>>>(                            \
        k_ph, v_ph, q_ph, alpha_ph, theta_ph, eta_ph, k_norm, q_norm, dk_ph, dv_ph, dq_ph,       \
        dalpha_ph, dtheta_ph, deta_ph, w_gates, (T*)d_kvq, dpre, n_tok, seq, d_model, num_heads)
        if (kvq_is_bf16) {
            if (ncl <= 1) NLH_LP_BWDW(__nv_bfloat16, 1); else if (ncl <= 2) NLH_LP_BWDW(__nv_bfloat16, 2); else NLH_LP_BWDW(__nv_bfloat16, 4);
        } else {
            if (ncl <= 1) NLH_LP_BWDW(float, 1); else if (ncl <= 2) NLH_LP_BWDW(float, 2); else NLH_LP_BWDW(float, 4);
        }
#undef NLH_LP_BWDW
        if (!check_launch("nlh_level_prep_backward")) return NLH_ERR_CUDA;
        gate_wgrad_kernel<<<grid, WG_THREADS, 0, st>>>(dpre, k_ph, v_ph, dw_partial, db_partial, n_tok, seq,
                                                       d_model, num_heads, lp_tok_per_cta(n_tok));
        return check_launch("nlh_level_prep_backward") ? NLH_OK : NLH_ERR_CUDA;
    }
#define NLH_LP_BWD(T, NE)                                                                        \
    level_prep_bwd_kernel<T, NE><<<grid, WR_THREADS, 0, st>>>(                                   \
        k_ph, v_ph, q_ph, alpha_ph, theta_ph, eta_ph, k_norm, q_norm, dk_ph, dv_ph, dq_ph,       \
        dalpha_ph, dtheta_ph, deta_ph, w_gates, (T*)d_kvq, dw_partial, db_partial, n_tok, seq,   \
        d_model, num_heads, lp_tok_per_cta(n_tok))
    if (kvq_is_bf16) {
        if (ne <= 1) NLH_LP_BWD(__nv_bfloat16, 1);
        else if (ne <= 2) NLH_LP_BWD(__nv_bfloat16, 2);
        else if (ne <= 4) NLH_LP_BWD(__nv_bfloat16, 4);
        else NLH_LP_BWD(__nv_bfloat16, 8);
    } else {
        if (ne <= 1) NLH_LP_BWD(float, 1);
        else if (ne <= 2) NLH_LP_BWD(float, 2);
        else if (ne <= 4) NLH_LP_BWD(float, 4);
        else NLH_LP_BWD(float, 8);
    }
#undef NLH_LP_BWD
    return check_launch("nlh_level_prep_backward") ? NLH_OK : NLH_ERR_CUDA;
}

static int fill_levels(CombineLevels& L, const float* y0, const float* y1, const float* y2,
                       const float* y3, int c0, int c1, int c2, int c3, int k, int S)
{
    if (k < 1 || k > WR_MAX_LEVELS) return NLH_ERR_INVALID_ARG;
    const float* ys[4] = {y0, y1, y2, y3};
    const int cs[4] = {c0, c1, c2, c3};
    for (int l = 0; l < WR_MAX_LEVELS; l++) {
        L.y[l] = l < k ? ys[l] : nullptr;
        L.c[l] = l < k ? cs[l] : 1;
        if (l < k && (ys[l] == nullptr || cs[l] <= 0 || S % cs[l] != 0)) return NLH_ERR_INVALID_ARG;
        L.cdiv[l] = make_fastdiv(L.c[l]);
    }
    L.sdiv = make_fastdiv(S);
    L.k = k;
    return NLH_OK;
}

int32_t nlh_mag_combine_forward(const float* x, const void* attn_proj, int32_t attn_is_bf16,
    const float* level_weights, const float* y0, const float* y1, const float* y2, const float* y3,
    int32_t c0, int32_t c1, int32_t c2, int32_t c3, int32_t k, float* out, int32_t batch,
    int32_t seq, int32_t d_model, int32_t num_heads)
{
    int rc = wr_check("nlh_mag_combine_forward", batch, seq, d_model, num_heads);
    if (rc != NLH_OK || batch == 0) return rc;
    CombineLevels L;
    if (fill_levels(L, y0, y1, y2, y3, c0, c1, c2, c3, k, seq) != NLH_OK) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_mag_combine_forward", "bad level list");
        return NLH_ERR_INVALID_ARG;
    }
    const int n_rows = batch * seq;
    const int need = (n_rows + CMB_WARPS - 1) / CMB_WARPS;
    const int grid = need < 148 * 8 ? need : 148 * 8;
    const int ncl = (d_model / 4 + 31) / 32;      // float4 chunks per lane, <= 8 because d_model <= 1024
    cudaStream_t st = current_stream();
#define NLH_CMB_FWD(T, NV)                                                                       \
    mag_combine_fwd_kernel<T, NV><<<grid, CMB_WARPS * 32, 0, st>>>(                                \
        x, (const T*)attn_proj, level_weights, L, out, batch, seq, d_model, num_heads)
    if (attn_is_bf16) {
        if (ncl <= 1) NLH_CMB_FWD(__nv_bfloat16, 1); else if (ncl <= 2) NLH_CMB_FWD(__nv_bfloat16, 2);
        else if (ncl <= 4) NLH_CMB_FWD(__nv_bfloat16, 4); else NLH_CMB_FWD(__nv_bfloat16, 8);
    } else {
        if (ncl <= 1) NLH_CMB_FWD(float, 1); else if (ncl <= 2) NLH_CMB_FWD(float, 2);
        else if (ncl <= 4) NLH_CMB_FWD(float, 4); else NLH_CMB_FWD(float, 8);
    }
#undef NLH_CMB_FWD
    return check_launch("nlh_mag_combine_forward") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_mag_combine_backward(const float* d_out, const void* attn_proj, int32_t attn_is_bf16,
    const float* level_weights, const float* y0, const float* y1, const float* y2, const float* y3,
    int32_t c0, int32_t c1, int32_t c2, int32_t c3, int32_t k, void* d_attn_proj, float* d_ycomb,
    float* dw_partial, int32_t n_partial_rows, float* dy0, float* dy1, float* dy2, float* dy3,
    int32_t batch, int32_t seq, int32_t d_model, int32_t num_heads)
{
    int rc = wr_check("nlh_mag_combine_backward", batch, seq, d_model, num_heads);
    if (rc != NLH_OK || batch == 0) return rc;
    CombineLevels L;
    if (n_partial_rows < 1 || fill_levels(L, y0, y1, y2, y3, c0, c1, c2, c3, k, seq) != NLH_OK) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_mag_combine_backward", "bad level list or partial rows");
        return NLH_ERR_INVALID_ARG;
    }
    cudaStream_t st = current_stream();
    CombineGrads G;
    float* dys[4] = {dy0, dy1, dy2, dy3};
    for (int l = 0; l < WR_MAX_LEVELS; l++) {
        G.dy[l] = (l < k) ? dys[l] : nullptr;
        if (G.dy[l] != nullptr && L.c[l] != 1) {
            record_status(NLH_ERR_INVALID_ARG, "nlh_mag_combine_backward", "dy output given for a pooled level");
            return NLH_ERR_INVALID_ARG;
        }
    }
    const int ncl = (d_model / 4 + 31) / 32;
#define NLH_CMB_BWD(T, NV)                                                                       \
    mag_combine_bwd_kernel<T, NV><<<n_partial_rows, CMB_WARPS * 32, 0, st>>>(                      \
        d_out, (const T*)attn_proj, level_weights, L, (T*)d_attn_proj, d_ycomb, dw_partial, G,  \
        batch, seq, d_model, num_heads)
    if (attn_is_bf16) {
        if (ncl <= 1) NLH_CMB_BWD(__nv_bfloat16, 1); else if (ncl <= 2) NLH_CMB_BWD(__nv_bfloat16, 2);
        else if (ncl <= 4) NLH_CMB_BWD(__nv_bfloat16, 4); else NLH_CMB_BWD(__nv_bfloat16, 8);
    } else {
        if (ncl <= 1) NLH_CMB_BWD(float, 1); else if (ncl <= 2) NLH_CMB_BWD(float, 2);
        else if (ncl <= 4) NLH_CMB_BWD(float, 4); else NLH_CMB_BWD(float, 8);
    }
#undef NLH_CMB_BWD
    return check_launch("nlh_mag_combine_backward") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_gate_grad_finish(const float* dw_partial, const float* db_partial, int32_t rows,
    int32_t d_model, float* g_w_gates, float* g_b_alpha, float* g_b_theta, float* g_b_eta)
{
    if (rows <= 0 || d_model <= 0 || !dw_partial || !db_partial || !g_w_gates) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_gate_grad_finish", "bad dimensions or NULL buffer");
        return NLH_ERR_INVALID_ARG;
    }
    const int cols = 3 * 2 * d_model;
    int slices = rows / 48;                       // about 48 rows per CTA, at most 16 slices
    slices = slices < 1 ? 1 : (slices > 16 ? 16 : slices);
    gate_grad_finish_kernel<<<dim3((cols + 255) / 256, slices), 256, 0, current_stream()>>>(
        dw_partial, db_partial, rows, cols, g_w_gates, g_b_alpha, g_b_theta, g_b_eta);
    return check_launch("nlh_gate_grad_finish") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_level_weight_grad_finish(const float* dw_partial, int32_t rows, int32_t k,
    const float* level_weights, float* g_logits)
{
    if (rows <= 0 || k <= 0 || k > WR_MAX_LEVELS || !dw_partial || !level_weights || !g_logits) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_level_weight_grad_finish", "bad dimensions or NULL buffer");
        return NLH_ERR_INVALID_ARG;
    }
    level_weight_grad_finish_kernel<<<1, 32 * WR_MAX_LEVELS, 0, current_stream()>>>(
        dw_partial, rows, k, level_weights, g_logits);
    return check_launch("nlh_level_weight_grad_finish") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_pool_to_heads(const float* d_ycomb, const float* level_weights, int32_t level,
    int32_t pool, float* dy_ph, float* sum_out, int32_t batch, int32_t seq, int32_t d_model,
    int32_t num_heads)
{
    int rc = wr_check("nlh_pool_to_heads", batch, seq, d_model, num_heads);
    if (rc != NLH_OK || batch == 0) return rc;
    if (pool <= 0 || seq % pool != 0 || level < 0 || level >= WR_MAX_LEVELS) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_pool_to_heads", "bad pool factor or level");
        return NLH_ERR_INVALID_ARG;
    }
    const long long n4 = (long long)batch * (seq / pool) * (d_model / 4);
    pool_to_heads_kernel<<<wr_grid(n4, 256), 256, 0, current_stream()>>>(
        d_ycomb, level_weights, level, pool, dy_ph, sum_out, batch, seq, d_model, num_heads);
    return check_launch("nlh_pool_to_heads") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_pool_heads(const float* src_sums, const float* level_weights, int32_t level,
    int32_t factor, float* dy_ph, float* sum_out, int32_t rows, int32_t src_seq, int32_t head_dim)
{
    if (rows < 0 || src_seq <= 0 || head_dim <= 0 || head_dim % 4 != 0 || factor <= 0 ||
        src_seq % factor != 0 || level < 0 || level >= WR_MAX_LEVELS) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_pool_heads", "bad dimensions, factor or level");
        return NLH_ERR_INVALID_ARG;
    }
    if (rows == 0) return NLH_OK;
    const long long n4 = (long long)rows * (src_seq / factor) * (head_dim / 4);
    pool_heads_kernel<<<wr_grid(n4, 256), 256, 0, current_stream()>>>(
        src_sums, level_weights, level, factor, dy_ph, sum_out, n4, head_dim / 4);
    return check_launch("nlh_pool_heads") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_mean_pool(const float* src, int32_t factor, float scale, void* out, int32_t out_is_bf16,
    float* sum_out, int32_t rows_out, int32_t d_model)
{
    if (rows_out < 0 || factor <= 0 || d_model <= 0 || d_model % 4 != 0 || !src || !out ||
        ((((uintptr_t)src | (uintptr_t)out | (uintptr_t)sum_out) & 15) != 0)) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_mean_pool", "bad dimensions, factor or alignment");
        return NLH_ERR_INVALID_ARG;
    }
    if (rows_out == 0) return NLH_OK;
    const long long n4 = (long long)rows_out * (d_model / 4);
    cudaStream_t st = current_stream();
    if (out_is_bf16)
        mean_pool_kernel<__nv_bfloat16><<<wr_grid(n4, 256), 256, 0, st>>>(src, factor, scale, (__nv_bfloat16*)out, sum_out, n4, d_model / 4);
    else
        mean_pool_kernel<float><<<wr_grid(n4, 256), 256, 0, st>>>(src, factor, scale, (float*)out, sum_out, n4, d_model / 4);
    return check_launch("nlh_mean_pool") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_unpool_sum(const void* g0, int32_t c0, int32_t g0_is_bf16, const void* g1, int32_t c1,
    int32_t g1_is_bf16, const void* g2, int32_t c2, int32_t g2_is_bf16, int32_t n_src, float* out,
    int32_t batch, int32_t seq, int32_t d_model)
{
    UnpoolSrc P;
    const void* gs[3] = {g0, g1, g2};
    const int cs[3] = {c0, c1, c2}, bs[3] = {g0_is_bf16, g1_is_bf16, g2_is_bf16};
    bool ok = batch >= 0 && seq > 0 && d_model > 0 && d_model % 8 == 0 && n_src >= 1 && n_src <= 3 && out &&
              (((uintptr_t)out & 15) == 0);
    for (int l = 0; l < 3; l++) {
        P.g[l] = l < n_src ? gs[l] : nullptr;
        P.c[l] = l < n_src ? cs[l] : 1;
        P.is_bf16[l] = bs[l];
        if (l < n_src && (gs[l] == nullptr || cs[l] <= 0 || seq % cs[l] != 0 || ((uintptr_t)gs[l] & 15) != 0)) ok = false;
        P.cdiv[l] = make_fastdiv(P.c[l]);
    }
    P.sdiv = make_fastdiv(seq > 0 ? seq : 1);
    P.n = n_src;
    if (!ok) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_unpool_sum", "bad dimensions, pool factors or alignment");
        return NLH_ERR_INVALID_ARG;
    }
    if (batch == 0) return NLH_OK;
    const long long n4 = (long long)batch * seq * (d_model / 4);
    unpool_sum_kernel<<<wr_grid(n4, 256), 256, 0, current_stream()>>>(P, out, n4, seq, d_model / 4);
    return check_launch("nlh_unpool_sum") ? NLH_OK : NLH_ERR_CUDA;
}

}  // extern "C"
