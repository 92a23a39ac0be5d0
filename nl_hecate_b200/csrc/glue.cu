// Stacked-block glue kernels: LayerNorm, cross-entropy, embedding gather / scatter-add.
//
// Drop-in entries keep the reference's signatures (core/src/cuda_ffi.rs:487-500, 523-538,
// 766-775; kernels core/kernels/layer_norm.cu, cross_entropy.cu, embedding.cu). The reference
// runs one CTA per row with shared-memory tree reductions and one atomicAdd per element for the
// LayerNorm parameter gradients; here
//   LayerNorm  : one WARP per row, the row lives in registers (one global read), shuffle
//                reductions only; backward is persistent, accumulates d_gamma/d_beta in
//                registers over all rows a warp visits and issues one atomicAdd per column
//                per CTA; optional bf16 copy of the output / bf16 upstream gradient so that the
//                bf16 GEMMs on either side need no separate cast pass.
//   cross-entropy : one pass online log-sum-exp per row; the additive entry keeps the
//                log-sum-exp so that the backward is a pure element-wise pass that can write
//                the gradient over the logits in place (bf16 or fp32).
//   embedding  : 16-byte gathers; scatter-add with vector atomics.
#include <cuda_bf16.h>
#include <math_constants.h>

#include "nlh_common.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {

constexpr int LN_MAXV = 8;          // most float4 chunks per lane: rows up to 32*8*4 = 1024 columns
constexpr int LN_WARPS = 8;

__device__ __forceinline__ float4 ld4f(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4f(const __nv_bfloat16* p)
{
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4bf(__nv_bfloat16* p, float4 v)
{
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&a);
    u.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

// ───────────────────────────── LayerNorm ─────────────────────────────────
// Optional operands that fold a residual block's neighbouring element-wise passes into the
// LayerNorm kernels (fast path only; every member may be NULL):
//   res_*      : second addend of the LayerNorm input, the kernels normalise x + res (forward and
//                backward; the sum is never written to memory);
//   add_in     : backward, fp32 [n, d] added to d_x (a gradient of x that arrives from another
//                consumer: the fan-in sum happens here instead of in a pass of its own);
//   d_x_bf16   : backward, bf16 copy of the INPUT gradient (without add_in) plus add_in_bf16 —
//                the gradient of a bf16 residual operand and its own fan-in.
struct LnExtra {
    const float* res_f32;
    const __nv_bfloat16* res_bf16;
    const float* add_in;
    __nv_bfloat16* d_x_bf16;
    const __nv_bfloat16* add_in_bf16;
};
__device__ __forceinline__ float4 ln_input(const float* __restrict__ x, const LnExtra& E, size_t off)
{
    float4 v = ld4f(x + off);
    if (E.res_f32) { const float4 r = ld4f(E.res_f32 + off); v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w; }
    if (E.res_bf16) { const float4 r = ld4f(E.res_bf16 + off); v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w; }
    return v;
}

// Fast path: d % 4 == 0, d <= 1024. Lane owns float4 chunks c = lane + 32*i, i < NV.
template <int NV>
__global__ void __launch_bounds__(LN_WARPS * 32) ln_fwd_kernel(
    const float* __restrict__ x, LnExtra E, const float* __restrict__ gamma, const float* __restrict__ beta,
    float* __restrict__ out, __nv_bfloat16* __restrict__ out_bf16, float* __restrict__ mean_cache,
    float* __restrict__ rstd_cache, int n, int d, float eps)
{
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
    if (row >= n) return;
    const int nv = d >> 2;
    float4 v[NV];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int c = lane + 32 * i;
        if (c < nv) { v[i] = ln_input(x, E, (size_t)row * d + 4 * c); s += (v[i].x + v[i].y) + (v[i].z + v[i].w); }
    }
    const float mean = warp_sum(s) / (float)d;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int c = lane + 32 * i;
        if (c < nv) {
            const float a = v[i].x - mean, b = v[i].y - mean, e = v[i].z - mean, f = v[i].w - mean;
            q += (a * a + b * b) + (e * e + f * f);
        }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(q) / (float)d + eps);
    if (lane == 0) {
        if (mean_cache) mean_cache[row] = mean;
        if (rstd_cache) rstd_cache[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int c = lane + 32 * i;
        if (c < nv) {
            const float4 g = ld4f(gamma + 4 * c), b = ld4f(beta + 4 * c);
            float4 o;
            o.x = g.x * (v[i].x - mean) * rstd + b.x;
            o.y = g.y * (v[i].y - mean) * rstd + b.y;
            o.z = g.z * (v[i].z - mean) * rstd + b.z;
            o.w = g.w * (v[i].w - mean) * rstd + b.w;
            if (out) *reinterpret_cast<float4*>(out + (size_t)row * d + 4 * c) = o;
            if (out_bf16) st4bf(out_bf16 + (size_t)row * d + 4 * c, o);
        }
    }
}

// Any d: one CTA per row, three passes over the row (L1/L2 resident).
__global__ void __launch_bounds__(256) ln_fwd_generic_kernel(
    const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
    float* __restrict__ out, __nv_bfloat16* __restrict__ out_bf16, float* __restrict__ mean_cache,
    float* __restrict__ rstd_cache, int n, int d, float eps)
{
    __shared__ float red[32];
    const int row = blockIdx.x;
    const float* xr = x + (size_t)row * d;
    float s = 0.f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) s += xr[j];
    const float mean = block_sum(s, red) / (float)d;
    float q = 0.f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) { const float a = xr[j] - mean; q += a * a; }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)d + eps);
    if (threadIdx.x == 0) {
        if (mean_cache) mean_cache[row] = mean;
        if (rstd_cache) rstd_cache[row] = rstd;
    }
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float o = gamma[j] * (xr[j] - mean) * rstd + beta[j];
        if (out) out[(size_t)row * d + j] = o;
        if (out_bf16) out_bf16[(size_t)row * d + j] = __float2bfloat16(o);
    }
}

// Upsampled gradient sources of the backward: gradients of mean-pooled copies of the LayerNorm
// output, g_l [rows / c_l, d] (fp32 or bf16), each contributing g_l[b, t / c_l, :] / c_l to row
// (b, t) (adjoint of core/kernels/pool_ops.cu mean pooling). seq = rows per sequence.
struct LnPooled {
    const void* g[3];
    int c[3];
    FastDiv cdiv[3];
    FastDiv sdiv;        // division by seq
    int is_bf16[3];
    int n;
    int seq;
};

// Backward, fast path. d_out = (fp32 part, may be NULL) + (bf16 part, may be NULL) + pooled parts.
// d_x = rstd/d * (d*dg - sum(dg) - x_hat*sum(dg*x_hat)), dg = d_out*gamma (core/src/mag.rs:421-449).
// Warp per row; the row's x_hat and output gradient stay in registers across the two warp sums.
template <int NV>
__device__ __forceinline__ float4 ln_bwd_dy(const float* __restrict__ d_out, const __nv_bfloat16* __restrict__ d_out_bf16,
                                            const LnPooled& P, const size_t ro, const size_t (&po)[3],
                                            const float (&pinv)[3], int c)
{
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    if (d_out) t = ld4f(d_out + ro + 4 * c);
    if (d_out_bf16) {
        const float4 w = ld4f(d_out_bf16 + ro + 4 * c);
        t.x += w.x; t.y += w.y; t.z += w.z; t.w += w.w;
    }
#pragma unroll
    for (int l = 0; l < 3; l++) {
        if (l < P.n) {
            const float4 w = P.is_bf16[l] ? ld4f((const __nv_bfloat16*)P.g[l] + po[l] + 4 * c)
                                          : ld4f((const float*)P.g[l] + po[l] + 4 * c);
            t.x += w.x * pinv[l]; t.y += w.y * pinv[l]; t.z += w.z * pinv[l]; t.w += w.w * pinv[l];
        }
    }
    return t;
}

template <int NV>
__global__ void __launch_bounds__(LN_WARPS * 32, 2) ln_bwd_kernel(
    const float* __restrict__ d_out, const __nv_bfloat16* __restrict__ d_out_bf16, LnPooled P,
    const float* __restrict__ x, LnExtra E, const float* __restrict__ gamma,
    const float* __restrict__ mean_cache, const float* __restrict__ rstd_cache,
    float* __restrict__ d_x, float* __restrict__ d_gamma, float* __restrict__ d_beta, int n, int d)
{
    constexpr int HV = (NV + 1) / 2;                  // chunks per lane handled per reduction round
    __shared__ float4 sred[LN_WARPS][32 * HV];   // [warp][chunk] for half of the chunks at a time
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nv = d >> 2;
    float4 ag[NV], ab[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) {
        ag[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float inv_d = 1.0f / (float)d;
    for (int row = blockIdx.x * LN_WARPS + warp; row < n; row += gridDim.x * LN_WARPS) {
        const float mean = mean_cache[row], rstd = rstd_cache[row];
        const size_t ro = (size_t)row * d;
        size_t po[3] = {0, 0, 0};
        float pinv[3] = {0.f, 0.f, 0.f};
        if (P.n > 0) {
            const int b = fd_div(row, P.sdiv), tt = row - b * P.seq;
#pragma unroll
            for (int l = 0; l < 3; l++)
                if (l < P.n) {
                    po[l] = ((size_t)b * fd_div(P.seq, P.cdiv[l]) + fd_div(tt, P.cdiv[l])) * d;
                    pinv[l] = 1.0f / (float)P.c[l];
                }
        }
        float4 xh[NV], dy[NV];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int c = lane + 32 * i;
            if (c < nv) {
                const float4 xv = ln_input(x, E, ro + 4 * c);
                const float4 t = ln_bwd_dy<NV>(d_out, d_out_bf16, P, ro, po, pinv, c);
                const float4 g = ld4f(gamma + 4 * c);
                const float4 h = make_float4((xv.x - mean) * rstd, (xv.y - mean) * rstd, (xv.z - mean) * rstd, (xv.w - mean) * rstd);
                xh[i] = h; dy[i] = t;
                ag[i].x += t.x * h.x; ag[i].y += t.y * h.y; ag[i].z += t.z * h.z; ag[i].w += t.w * h.w;
                ab[i].x += t.x; ab[i].y += t.y; ab[i].z += t.z; ab[i].w += t.w;
                const float a = t.x * g.x, b = t.y * g.y, e = t.z * g.z, f = t.w * g.w;
                s1 += (a + b) + (e + f);
                s2 += (a * h.x + b * h.y) + (e * h.z + f * h.w);
            }
        }
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        const float k = rstd * inv_d;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int c = lane + 32 * i;
            if (c < nv) {
                const float4 g = ld4f(gamma + 4 * c);
                float4 o;
                o.x = k * ((float)d * dy[i].x * g.x - s1 - xh[i].x * s2);
                o.y = k * ((float)d * dy[i].y * g.y - s1 - xh[i].y * s2);
                o.z = k * ((float)d * dy[i].z * g.z - s1 - xh[i].z * s2);
                o.w = k * ((float)d * dy[i].w * g.w - s1 - xh[i].w * s2);
                if (E.d_x_bf16) {
                    float4 ob = o;
                    if (E.add_in_bf16) {
                        const float4 r = ld4f(E.add_in_bf16 + ro + 4 * c);
                        ob.x += r.x; ob.y += r.y; ob.z += r.z; ob.w += r.w;
                    }
                    st4bf(E.d_x_bf16 + ro + 4 * c, ob);
                }
                if (E.add_in) {
                    const float4 r = ld4f(E.add_in + ro + 4 * c);
                    o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
                }
                *reinterpret_cast<float4*>(d_x + ro + 4 * c) = o;
            }
        }
    }
    // cross-warp sums of the parameter gradients, HV chunks per lane per round, gamma then beta
#pragma unroll
    for (int which = 0; which < 2; which++) {
#pragma unroll
        for (int half = 0; half * HV < NV; half++) {
            __syncthreads();
#pragma unroll
            for (int i = 0; i < HV; i++)
                if (half * HV + i < NV) sred[warp][lane + 32 * i] = which == 0 ? ag[half * HV + i] : ab[half * HV + i];
            __syncthreads();
            float* dst = which == 0 ? d_gamma : d_beta;
            for (int cc = threadIdx.x; cc < 32 * HV; cc += blockDim.x) {
                const int c = half * (32 * HV) + cc;     // chunk index lane + 32*i
                if (c < nv && (cc >> 5) + half * HV < NV) {
                    float4 t = sred[0][cc];
#pragma unroll
                    for (int w = 1; w < LN_WARPS; w++) {
                        t.x += sred[w][cc].x; t.y += sred[w][cc].y; t.z += sred[w][cc].z; t.w += sred[w][cc].w;
                    }
                    atomicAdd(dst + 4 * c + 0, t.x);
                    atomicAdd(dst + 4 * c + 1, t.y);
                    atomicAdd(dst + 4 * c + 2, t.z);
                    atomicAdd(dst + 4 * c + 3, t.w);
                }
            }
        }
    }
}

// Any d: one CTA per row; parameter gradients by one atomicAdd per element like the reference.
__global__ void __launch_bounds__(256) ln_bwd_generic_kernel(
    const float* __restrict__ d_out, const __nv_bfloat16* __restrict__ d_out_bf16,
    const float* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ mean_cache, const float* __restrict__ rstd_cache,
    float* __restrict__ d_x, float* __restrict__ d_gamma, float* __restrict__ d_beta, int n, int d)
{
    __shared__ float red[32];
    const int row = blockIdx.x;
    const size_t ro = (size_t)row * d;
    const float mean = mean_cache[row], rstd = rstd_cache[row];
    auto dyv = [&](int j) {
        float t = d_out ? d_out[ro + j] : 0.f;
        if (d_out_bf16) t += __bfloat162float(d_out_bf16[ro + j]);
        return t;
    };
    float s1 = 0.f, s2 = 0.f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float xh = (x[ro + j] - mean) * rstd, dg = dyv(j) * gamma[j];
        s1 += dg; s2 += dg * xh;
    }
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    const float k = rstd / (float)d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float xh = (x[ro + j] - mean) * rstd, dy = dyv(j);
        d_x[ro + j] = k * ((float)d * dy * gamma[j] - s1 - xh * s2);
        atomicAdd(d_gamma + j, dy * xh);
        atomicAdd(d_beta + j, dy);
    }
}

// ───────────────────────────── cross-entropy ─────────────────────────────
__device__ __forceinline__ float ce_ld(const float* p) { return *p; }
__device__ __forceinline__ float ce_ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// (max, sum of exp(x - max)) pairs merge associatively.
// 2^x with the hardware approximation, flushing denormals: one instruction.
__device__ __forceinline__ float ex2_ftz(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr float CE_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2)
{
    const float mm = fmaxf(m, m2);
    if (mm == -CUDART_INF_F) { m = mm; s = 0.f; return; }
    s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
    m = mm;
}

// One CTA per row: log-sum-exp in one pass over the row. Not inlined: the cross-entropy backward
// calls it only when no stored log-sum-exp is given, and its 32-value register block must not
// raise the register count of that kernel's main path.
template <typename T>
__device__ __noinline__ float row_lse(const T* __restrict__ row, int vocab, float* red_m, float* red_s)
{
    float m = -CUDART_INF_F, s = 0.f;
    if (sizeof(T) == 2 && (vocab & 7) == 0 && ((uintptr_t)row & 15) == 0) {
        // four 16-byte loads per thread in flight, one running-maximum update per 32 values
        const uint4* r4 = reinterpret_cast<const uint4*>(row);
        const int nvec = vocab >> 3;
        for (int j0 = threadIdx.x; j0 < nvec; j0 += 4 * blockDim.x) {
            uint4 u[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int jj = j0 + q * blockDim.x;
                u[q] = jj < nvec ? r4[jj] : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);   // -inf pairs
            }
            float f[32];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const unsigned w[4] = {u[q].x, u[q].y, u[q].z, u[q].w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
                    f[8 * q + 2 * e] = t.x; f[8 * q + 2 * e + 1] = t.y;
                }
            }
            float lm = f[0];
#pragma unroll
            for (int q = 1; q < 32; q++) lm = fmaxf(lm, f[q]);
            const float mm = fmaxf(m, lm);
            if (mm == -CUDART_INF_F) continue;
            const float nb = -mm * CE_LOG2E;             // e^(f - mm) = 2^(f log2e - mm log2e): one FMA + ex2
            float ls = 0.f;
#pragma unroll
            for (int q = 0; q < 32; q++) ls += ex2_ftz(fmaf(f[q], CE_LOG2E, nb));
            s = s * ex2_ftz(fmaf(m, CE_LOG2E, nb)) + ls;
            m = mm;
        }
    } else {
        for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
            const float x = ce_ld(row + j);
            const float mm = fmaxf(m, x);
            s = s * __expf(m - mm) + __expf(x - mm);
            m = mm;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        lse_merge(m, s, m2, s2);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) { red_m[warp] = m; red_s[warp] = s; }
    __syncthreads();
    m = red_m[0];
    for (int w = 1; w < nw; w++) m = fmaxf(m, red_m[w]);
    if (m == -CUDART_INF_F) { __syncthreads(); return m; }
    s = 0.f;
    for (int w = 0; w < nw; w++) s += red_s[w] * ex2_ftz((red_m[w] - m) * CE_LOG2E);
    __syncthreads();
    return m + logf(s);
}

// loss_sum += lse - logit[target] for valid targets; lse_out (optional) keeps the row's log-sum-exp.
template <typename T>
__global__ void __launch_bounds__(256) ce_fwd_kernel(const T* __restrict__ logits,
    const int* __restrict__ targets, float* __restrict__ loss_sum, float* __restrict__ lse_out,
    int* __restrict__ valid_count, int vocab)
{
    __shared__ float red_m[32], red_s[32];
    const int t = blockIdx.x;
    const T* row = logits + (size_t)t * vocab;
    const int target = targets[t];
    const bool valid = target >= 0 && target < vocab;
    if (!valid && lse_out == nullptr) return;
    const float lse = row_lse(row, vocab, red_m, red_s);
    if (threadIdx.x == 0) {
        if (lse_out) lse_out[t] = lse;
        if (valid) {
            atomicAdd(loss_sum, lse - ce_ld(row + target));
            if (valid_count) atomicAdd(valid_count, 1);
        }
    }
}

// d_logits = (softmax - onehot) * inv_count * (*grad_scale); rows with invalid targets are zero.
// lse == NULL: the log-sum-exp is recomputed here. d_logits may alias logits.
template <typename T>
__global__ void __launch_bounds__(256) ce_bwd_kernel(const T* logits,
    const int* __restrict__ targets, const float* __restrict__ lse_in, const float* __restrict__ grad_scale,
    T* d_logits, int vocab, float inv_count)
{
    __shared__ float red_m[32], red_s[32];
    const int t = blockIdx.x;
    const T* row = logits + (size_t)t * vocab;
    T* drow = d_logits + (size_t)t * vocab;
    const int target = targets[t];
    if (target < 0 || target >= vocab) {
        for (int j = threadIdx.x; j < vocab; j += blockDim.x) drow[j] = T(0.f);
        return;
    }
    const float lse = lse_in ? lse_in[t] : row_lse(row, vocab, red_m, red_s);
    const float sc = inv_count * (grad_scale ? *grad_scale : 1.0f);
    if (sizeof(T) == 2 && (vocab & 7) == 0 && (((uintptr_t)row | (uintptr_t)drow) & 15) == 0) {
        const uint4* r4 = reinterpret_cast<const uint4*>(row);
        uint4* d4 = reinterpret_cast<uint4*>(drow);
        for (int j = threadIdx.x; j < (vocab >> 3); j += blockDim.x) {
            const uint4 u = r4[j];
            unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[q]));
                const int c = 8 * j + 2 * q;
                const float a = (__expf(f.x - lse) - (c == target ? 1.f : 0.f)) * sc;
                const float b = (__expf(f.y - lse) - (c + 1 == target ? 1.f : 0.f)) * sc;
                const __nv_bfloat162 o = __floats2bfloat162_rn(a, b);
                w[q] = *reinterpret_cast<const unsigned*>(&o);
            }
            d4[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        for (int j = threadIdx.x; j < vocab; j += blockDim.x)
            drow[j] = T((__expf(ce_ld(row + j) - lse) - (j == target ? 1.f : 0.f)) * sc);
    }
}

// ───────────────────────────── embedding ─────────────────────────────────
__global__ void __launch_bounds__(128) embedding_gather_kernel(const float* __restrict__ w_embed,
    const int* __restrict__ ids, float* __restrict__ out, int d)
{
    const int t = blockIdx.x;
    const float* src = w_embed + (size_t)ids[t] * d;
    float* dst = out + (size_t)t * d;
    if ((d & 3) == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
        for (int j = threadIdx.x; j < (d >> 2); j += blockDim.x)
            reinterpret_cast<float4*>(dst)[j] = reinterpret_cast<const float4*>(src)[j];
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) dst[j] = src[j];
    }
}

__global__ void __launch_bounds__(128) embedding_scatter_add_kernel(const float* __restrict__ d_embedded,
    const int* __restrict__ ids, float* __restrict__ d_embed, int d)
{
    const int t = blockIdx.x;
    const float* src = d_embedded + (size_t)t * d;
    float* dst = d_embed + (size_t)ids[t] * d;
    if ((d & 3) == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
        for (int j = threadIdx.x; j < (d >> 2); j += blockDim.x)
            atomicAdd(reinterpret_cast<float4*>(dst) + j, reinterpret_cast<const float4*>(src)[j]);
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) atomicAdd(dst + j, src[j]);
    }
}

}  // namespace nlh

using namespace nlh;

static bool ln_fast_ok(const void* a, const void* b, const void* c, const void* e, const void* f,
                       const void* g, int d)
{
    const uintptr_t u = (uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)e | (uintptr_t)f | (uintptr_t)g;
    return (d & 3) == 0 && d <= 128 * LN_MAXV && (u & 15) == 0;
}

static bool ln_extra_any(const LnExtra& E)
{
    return E.res_f32 || E.res_bf16 || E.add_in || E.d_x_bf16 || E.add_in_bf16;
}
static bool ln_extra_aligned(const LnExtra& E, int d)
{
    const uintptr_t u = (uintptr_t)E.res_f32 | (uintptr_t)E.res_bf16 | (uintptr_t)E.add_in |
                        (uintptr_t)E.d_x_bf16 | (uintptr_t)E.add_in_bf16;
    return (u & 15) == 0 && (d & 7) == 0;
}

static int ln_forward(const char* where, const float* x, const float* gamma, const float* beta,
                      float* out, __nv_bfloat16* out_bf16, float* mean_cache, float* rstd_cache,
                      int n, int d, float eps, const LnExtra* extra = nullptr)
{
    LnExtra E = {nullptr, nullptr, nullptr, nullptr, nullptr};
    if (extra) E = *extra;
    if (n < 0 || d <= 0 || !x || !gamma || !beta || (!out && !out_bf16)) {
        record_status(NLH_ERR_INVALID_ARG, where, "bad dimensions or NULL pointer");
        return NLH_ERR_INVALID_ARG;
    }
    if (n == 0) return NLH_OK;
    cudaStream_t st = current_stream();
    const bool fast = ln_fast_ok(x, gamma, beta, out, out_bf16, nullptr, d) && (!out_bf16 || (d & 7) == 0);
    if (ln_extra_any(E) && !(fast && ln_extra_aligned(E, d))) {
        record_status(NLH_ERR_UNSUPPORTED, where, "fused operands need d % 8 == 0, d <= 1024 and 16-byte aligned buffers");
        return NLH_ERR_UNSUPPORTED;
    }
    if (fast) {
        const int grid = (n + LN_WARPS - 1) / LN_WARPS;
        const int nv = (d / 4 + 31) / 32;
#define NLH_LN_FWD(NV) ln_fwd_kernel<NV><<<grid, LN_WARPS * 32, 0, st>>>(x, E, gamma, beta, out, out_bf16, mean_cache, rstd_cache, n, d, eps)
        if (nv <= 1) NLH_LN_FWD(1); else if (nv <= 2) NLH_LN_FWD(2); else if (nv <= 4) NLH_LN_FWD(4); else NLH_LN_FWD(8);
#undef NLH_LN_FWD
    } else {
        ln_fwd_generic_kernel<<<n, 256, 0, st>>>(x, gamma, beta, out, out_bf16, mean_cache, rstd_cache, n, d, eps);
    }
    return check_launch(where) ? NLH_OK : NLH_ERR_CUDA;
}

static int ln_backward(const char* where, const float* d_out, const __nv_bfloat16* d_out_bf16,
                       const float* x, const float* gamma, const float* mean_cache,
                       const float* rstd_cache, float* d_x, float* d_gamma, float* d_beta, int n, int d,
                       const LnPooled* pooled = nullptr, const LnExtra* extra = nullptr)
{
    LnExtra E = {nullptr, nullptr, nullptr, nullptr, nullptr};
    if (extra) E = *extra;
    LnPooled P;
    P.n = 0; P.seq = 1; P.sdiv = make_fastdiv(1);
    for (int l = 0; l < 3; l++) { P.g[l] = nullptr; P.c[l] = 1; P.is_bf16[l] = 0; P.cdiv[l] = make_fastdiv(1); }
    if (pooled) P = *pooled;
    if (n < 0 || d <= 0 || (!d_out && !d_out_bf16 && P.n == 0) || !x || !gamma || !mean_cache || !rstd_cache ||
        !d_x || !d_gamma || !d_beta) {
        record_status(NLH_ERR_INVALID_ARG, where, "bad dimensions or NULL pointer");
        return NLH_ERR_INVALID_ARG;
    }
    if (n == 0) return NLH_OK;
    cudaStream_t st = current_stream();
    const bool fast = ln_fast_ok(x, gamma, d_out, d_out_bf16, d_x, nullptr, d) && (!d_out_bf16 || (d & 7) == 0);
    if ((P.n > 0 && !(fast && (d & 7) == 0)) || (ln_extra_any(E) && !(fast && ln_extra_aligned(E, d)))) {
        record_status(NLH_ERR_UNSUPPORTED, where, "pooled gradient sources and fused operands need d % 8 == 0, d <= 1024 and 16-byte aligned buffers");
        return NLH_ERR_UNSUPPORTED;
    }
    if (fast) {
        const int need = (n + LN_WARPS - 1) / LN_WARPS;
        const int nv = (d / 4 + 31) / 32;
        // persistent: a few CTAs per SM, each warp walks rows so that the parameter gradients
        // are reduced once per CTA
        const int grid = need < 148 * 2 ? need : 148 * 2;
#define NLH_LN_BWD(NV) ln_bwd_kernel<NV><<<grid, LN_WARPS * 32, 0, st>>>(d_out, d_out_bf16, P, x, E, gamma, mean_cache, rstd_cache, d_x, d_gamma, d_beta, n, d)
        if (nv <= 1) NLH_LN_BWD(1); else if (nv <= 2) NLH_LN_BWD(2); else if (nv <= 4) NLH_LN_BWD(4); else NLH_LN_BWD(8);
#undef NLH_LN_BWD
    } else {
        ln_bwd_generic_kernel<<<n, 256, 0, st>>>(d_out, d_out_bf16, x, gamma, mean_cache, rstd_cache, d_x, d_gamma, d_beta, n, d);
    }
    return check_launch(where) ? NLH_OK : NLH_ERR_CUDA;
}

extern "C" {

void layer_norm_forward_cuda(const float* x, const float* gamma, const float* beta, float* out,
    float* mean_cache, float* rstd_cache, int32_t n, int32_t d, float eps)
{
    ln_forward("layer_norm_forward_cuda", x, gamma, beta, out, nullptr, mean_cache, rstd_cache, n, d, eps);
}

void layer_norm_backward_cuda(const float* d_out, const float* x, const float* gamma,
    const float* mean_cache, const float* rstd_cache, float* d_x, float* d_gamma, float* d_beta,
    int32_t n, int32_t d)
{
    ln_backward("layer_norm_backward_cuda", d_out, nullptr, x, gamma, mean_cache, rstd_cache, d_x, d_gamma, d_beta, n, d);
}

int32_t nlh_layer_norm_forward(const float* x, const float* gamma, const float* beta, float* out_f32,
    uint16_t* out_bf16, float* mean_cache, float* rstd_cache, int32_t n, int32_t d, float eps)
{
    return ln_forward("nlh_layer_norm_forward", x, gamma, beta, out_f32, (__nv_bfloat16*)out_bf16,
                      mean_cache, rstd_cache, n, d, eps);
}

int32_t nlh_layer_norm_backward(const float* d_out_f32, const uint16_t* d_out_bf16, const float* x,
    const float* gamma, const float* mean_cache, const float* rstd_cache, float* d_x, float* d_gamma,
    float* d_beta, int32_t n, int32_t d)
{
    return ln_backward("nlh_layer_norm_backward", d_out_f32, (const __nv_bfloat16*)d_out_bf16, x, gamma,
                       mean_cache, rstd_cache, d_x, d_gamma, d_beta, n, d);
}

int32_t nlh_layer_norm_backward_pooled(const float* d_out_f32, const uint16_t* d_out_bf16,
    const void* g0, int32_t c0, int32_t g0_is_bf16, const void* g1, int32_t c1, int32_t g1_is_bf16,
    const void* g2, int32_t c2, int32_t g2_is_bf16, int32_t n_src, int32_t seq, const float* x,
    const float* gamma, const float* mean_cache, const float* rstd_cache, float* d_x, float* d_gamma,
    float* d_beta, int32_t n, int32_t d)
{
    LnPooled P;
    const void* gs[3] = {g0, g1, g2};
    const int cs[3] = {c0, c1, c2}, bs[3] = {g0_is_bf16, g1_is_bf16, g2_is_bf16};
    bool ok = n_src >= 0 && n_src <= 3 && seq > 0 && n % seq == 0;
    for (int l = 0; l < 3; l++) {
        P.g[l] = l < n_src ? gs[l] : nullptr;
        P.c[l] = l < n_src ? cs[l] : 1;
        P.is_bf16[l] = bs[l];
        if (l < n_src && (gs[l] == nullptr || cs[l] <= 0 || seq % cs[l] != 0 || ((uintptr_t)gs[l] & 15) != 0)) ok = false;
        P.cdiv[l] = make_fastdiv(P.c[l]);
    }
    P.n = n_src; P.seq = seq; P.sdiv = make_fastdiv(seq > 0 ? seq : 1);
    if (!ok) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_layer_norm_backward_pooled", "bad pooled sources, pool factors or alignment");
        return NLH_ERR_INVALID_ARG;
    }
    return ln_backward("nlh_layer_norm_backward_pooled", d_out_f32, (const __nv_bfloat16*)d_out_bf16, x, gamma,
                       mean_cache, rstd_cache, d_x, d_gamma, d_beta, n, d, &P);
}

int32_t nlh_layer_norm_residual_forward(const float* x, const void* res, int32_t res_is_bf16,
    const float* gamma, const float* beta, float* out_f32, uint16_t* out_bf16, float* mean_cache,
    float* rstd_cache, int32_t n, int32_t d, float eps)
{
    LnExtra E = {nullptr, nullptr, nullptr, nullptr, nullptr};
    if (res) { if (res_is_bf16) E.res_bf16 = (const __nv_bfloat16*)res; else E.res_f32 = (const float*)res; }
    return ln_forward("nlh_layer_norm_residual_forward", x, gamma, beta, out_f32, (__nv_bfloat16*)out_bf16,
                      mean_cache, rstd_cache, n, d, eps, &E);
}

int32_t nlh_layer_norm_backward_fused(const float* d_out_f32, const uint16_t* d_out_bf16,
    const void* g0, int32_t c0, int32_t g0_is_bf16, const void* g1, int32_t c1, int32_t g1_is_bf16,
    const void* g2, int32_t c2, int32_t g2_is_bf16, int32_t n_src, int32_t seq, const float* x,
    const void* res, int32_t res_is_bf16, const float* add_in, const float* gamma,
    const float* mean_cache, const float* rstd_cache, float* d_x, uint16_t* d_x_bf16,
    const uint16_t* add_in_bf16, float* d_gamma, float* d_beta, int32_t n, int32_t d)
{
    LnPooled P;
    const void* gs[3] = {g0, g1, g2};
    const int cs[3] = {c0, c1, c2}, bs[3] = {g0_is_bf16, g1_is_bf16, g2_is_bf16};
    bool ok = n_src >= 0 && n_src <= 3 && seq > 0 && n % seq == 0 && (d_x_bf16 || !add_in_bf16);
    for (int l = 0; l < 3; l++) {
        P.g[l] = l < n_src ? gs[l] : nullptr;
        P.c[l] = l < n_src ? cs[l] : 1;
        P.is_bf16[l] = bs[l];
        if (l < n_src && (gs[l] == nullptr || cs[l] <= 0 || seq % cs[l] != 0 || ((uintptr_t)gs[l] & 15) != 0)) ok = false;
        P.cdiv[l] = make_fastdiv(P.c[l]);
    }
    P.n = n_src; P.seq = seq; P.sdiv = make_fastdiv(seq > 0 ? seq : 1);
    if (!ok) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_layer_norm_backward_fused", "bad pooled sources, pool factors, alignment or operands");
        return NLH_ERR_INVALID_ARG;
    }
    LnExtra E = {nullptr, nullptr, add_in, (__nv_bfloat16*)d_x_bf16, (const __nv_bfloat16*)add_in_bf16};
    if (res) { if (res_is_bf16) E.res_bf16 = (const __nv_bfloat16*)res; else E.res_f32 = (const float*)res; }
    return ln_backward("nlh_layer_norm_backward_fused", d_out_f32, (const __nv_bfloat16*)d_out_bf16, x, gamma,
                       mean_cache, rstd_cache, d_x, d_gamma, d_beta, n, d, &P, &E);
}

void embedding_gather_cuda(const float* w_embed, const int32_t* input_ids, float* output,
    int32_t seq_len, int32_t d)
{
    if (seq_len <= 0 || d <= 0) return;
    embedding_gather_kernel<<<seq_len, 128, 0, current_stream()>>>(w_embed, input_ids, output, d);
    check_launch("embedding_gather_cuda");
}

void embedding_scatter_add_cuda(const float* d_embedded, const int32_t* input_ids, float* d_embed,
    int32_t seq_len, int32_t d)
{
    if (seq_len <= 0 || d <= 0) return;
    embedding_scatter_add_kernel<<<seq_len, 128, 0, current_stream()>>>(d_embedded, input_ids, d_embed, d);
    check_launch("embedding_scatter_add_cuda");
}

void cross_entropy_forward_cuda(const float* logits, const int32_t* target_ids, float* loss_out,
    int32_t seq_len, int32_t vocab)
{
    cudaStream_t st = current_stream();
    cudaMemsetAsync(loss_out, 0, sizeof(float), st);   // the reference entry zeroes it too
    if (seq_len <= 0 || vocab <= 0) return;
    ce_fwd_kernel<float><<<seq_len, 256, 0, st>>>(logits, target_ids, loss_out, nullptr, nullptr, vocab);
    check_launch("cross_entropy_forward_cuda");
}

void cross_entropy_backward_cuda(const float* logits, const int32_t* target_ids, float* d_logits,
    int32_t seq_len, int32_t vocab, float inv_count)
{
    if (seq_len <= 0 || vocab <= 0) return;
    ce_bwd_kernel<float><<<seq_len, 256, 0, current_stream()>>>(logits, target_ids, nullptr, nullptr,
                                                              d_logits, vocab, inv_count);
    check_launch("cross_entropy_backward_cuda");
}

int32_t nlh_cross_entropy_forward(const void* logits, int32_t logits_is_bf16, const int32_t* target_ids,
    float* loss_sum, float* lse, int32_t* valid_count, int32_t n, int32_t vocab)
{
    if (n < 0 || vocab <= 0 || !logits || !target_ids || !loss_sum) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_cross_entropy_forward", "bad dimensions or NULL pointer");
        return NLH_ERR_INVALID_ARG;
    }
    if (n == 0) return NLH_OK;
    cudaStream_t st = current_stream();
    if (logits_is_bf16)
        ce_fwd_kernel<__nv_bfloat16><<<n, 256, 0, st>>>((const __nv_bfloat16*)logits, target_ids, loss_sum, lse, valid_count, vocab);
    else
        ce_fwd_kernel<float><<<n, 256, 0, st>>>((const float*)logits, target_ids, loss_sum, lse, valid_count, vocab);
    return check_launch("nlh_cross_entropy_forward") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_cross_entropy_backward(const void* logits, int32_t logits_is_bf16, const int32_t* target_ids,
    const float* lse, const float* grad_scale, void* d_logits, int32_t n, int32_t vocab, float inv_count)
{
    if (n < 0 || vocab <= 0 || !logits || !target_ids || !d_logits) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_cross_entropy_backward", "bad dimensions or NULL pointer");
        return NLH_ERR_INVALID_ARG;
    }
    if (n == 0) return NLH_OK;
    cudaStream_t st = current_stream();
    if (logits_is_bf16)
        ce_bwd_kernel<__nv_bfloat16><<<n, 256, 0, st>>>((const __nv_bfloat16*)logits, target_ids, lse, grad_scale, (__nv_bfloat16*)d_logits, vocab, inv_count);
    else
        ce_bwd_kernel<float><<<n, 256, 0, st>>>((const float*)logits, target_ids, lse, grad_scale, (float*)d_logits, vocab, inv_count);
    return check_launch("nlh_cross_entropy_backward") ? NLH_OK : NLH_ERR_CUDA;
}

}  // extern "C"
