// AdamW outer-parameter step, gradient-norm partials and clip, for sm_100a.
//
// HBM-bound element-wise work: 16 B read + 12 B written per parameter. Every
// kernel uses 16-byte vector accesses when the pointers allow it and a grid of
// (a multiple of) 148 SMs × resident CTAs with a grid-stride loop.
//
// Entry points with the reference's signatures replace core/kernels/adamw.cu
// (declared in core/src/cuda_ffi.rs:674-716); nlh_adamw_multi_tensor is the
// single-launch form of the per-tensor loop in
// core/src/gpu_stacked_optimizer.rs:522-683.
#include "nlh_common.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {

constexpr int AW_THREADS = 256;

__device__ __forceinline__ void adamw_elem(float& w, float g, float& m, float& v, float lr,
                                           float b1, float b2, float eps, float bc1, float bc2,
                                           float wd)
{
    m = b1 * m + (1.0f - b1) * g;
    v = b2 * v + (1.0f - b2) * g * g;
    const float mh = m * bc1;
    const float vh = v * bc2;
    w -= lr * (mh / (sqrtf(vh) + eps) + wd * w);
}

__global__ void __launch_bounds__(AW_THREADS) adamw_vec4_kernel(
    float4* __restrict__ w, const float4* __restrict__ g, float4* __restrict__ m,
    float4* __restrict__ v, long long n4, float lr, float b1, float b2, float eps, float bc1,
    float bc2, float wd)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        float4 wi = w[i], mi = m[i], vi = v[i];
        const float4 gi = g[i];
        adamw_elem(wi.x, gi.x, mi.x, vi.x, lr, b1, b2, eps, bc1, bc2, wd);
        adamw_elem(wi.y, gi.y, mi.y, vi.y, lr, b1, b2, eps, bc1, bc2, wd);
        adamw_elem(wi.z, gi.z, mi.z, vi.z, lr, b1, b2, eps, bc1, bc2, wd);
        adamw_elem(wi.w, gi.w, mi.w, vi.w, lr, b1, b2, eps, bc1, bc2, wd);
        w[i] = wi; m[i] = mi; v[i] = vi;
    }
}

__global__ void __launch_bounds__(AW_THREADS) adamw_scalar_kernel(
    float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m,
    float* __restrict__ v, long long start, long long n, float lr, float b1, float b2, float eps,
    float bc1, float bc2, float wd)
{
    for (long long i = start + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        float wi = w[i], mi = m[i], vi = v[i];
        adamw_elem(wi, g[i], mi, vi, lr, b1, b2, eps, bc1, bc2, wd);
        w[i] = wi; m[i] = mi; v[i] = vi;
    }
}

// One partial per 256 consecutive elements (the contract of grad_norm_sq_cuda:
// *out_num_blocks = ceil(n/256) partial sums). One warp per 256-element block,
// 8 elements per lane, shuffle-reduced: deterministic.
template <bool DOT>
__global__ void __launch_bounds__(AW_THREADS) partial256_kernel(
    const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ partial,
    long long n, long long nblocks)
{
    const int lane = threadIdx.x & 31;
    const long long warps_per_grid = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
         blk < nblocks; blk += warps_per_grid) {
        const long long base = blk * 256;
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < 8; r++) {
            const long long i = base + r * 32 + lane;
            if (i < n) {
                const float x = a[i];
                s += DOT ? x * b[i] : x * x;
            }
        }
        s = warp_sum(s);
        if (lane == 0) partial[blk] = s;
    }
}

__global__ void __launch_bounds__(AW_THREADS) scale_kernel(float* __restrict__ g,
                                                           const float* __restrict__ scale_ptr,
                                                           float scale_val, long long n)
{
    float scale = scale_val;
    if (scale_ptr != nullptr) {
        scale = *scale_ptr;
        if (scale >= 1.0f) return;  // conditional form: no-op unless clipping is active
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        g[i] *= scale;
}

__global__ void __launch_bounds__(AW_THREADS) reduce_partials_clip_kernel(
    const float* __restrict__ partial, long long total, float max_norm, float* out_norm,
    float* out_scale)
{
    __shared__ float red[32];
    float acc = 0.0f;
    for (long long i = threadIdx.x; i < total; i += blockDim.x) acc += partial[i];
    const float tot = block_sum(acc, red);
    if (threadIdx.x == 0) {
        const float norm = sqrtf(tot);
        *out_norm = norm;
        *out_scale = (norm > max_norm && max_norm > 0.0f) ? (max_norm / norm) : 1.0f;
    }
}

// ── multi-tensor AdamW over a flat arena ──────────────────────────────────
// The arena is cut into fixed chunks; chunk c belongs to tensor chunk_tensor[c]
// and covers [chunk_start[c], chunk_start[c] + chunk_len[c]).
__global__ void __launch_bounds__(AW_THREADS) adamw_multi_kernel(
    float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m,
    float* __restrict__ v, const nlh_adamw_tensor_desc* __restrict__ descs,
    const int* __restrict__ chunk_tensor, const long long* __restrict__ chunk_start,
    const int* __restrict__ chunk_len, int n_chunks, const float* __restrict__ grad_scale_ptr,
    float lr, float b1, float b2, float eps)
{
    const float gs = (grad_scale_ptr != nullptr) ? fminf(*grad_scale_ptr, 1.0f) : 1.0f;
    for (int c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const nlh_adamw_tensor_desc ds = descs[chunk_tensor[c]];
        if (!ds.active) continue;
        const long long s0 = chunk_start[c];
        const int len = chunk_len[c];
        const float tlr = lr * ds.lr_scale;
        if ((s0 & 3) == 0 && (len & 3) == 0) {
            float4* w4 = reinterpret_cast<float4*>(w + s0);
            const float4* g4 = reinterpret_cast<const float4*>(g + s0);
            float4* m4 = reinterpret_cast<float4*>(m + s0);
            float4* v4 = reinterpret_cast<float4*>(v + s0);
            for (int i = threadIdx.x; i < (len >> 2); i += blockDim.x) {
                float4 wi = w4[i], mi = m4[i], vi = v4[i];
                float4 gi = g4[i];
                gi.x *= gs; gi.y *= gs; gi.z *= gs; gi.w *= gs;
                adamw_elem(wi.x, gi.x, mi.x, vi.x, tlr, b1, b2, eps, ds.bc1_inv, ds.bc2_inv, ds.weight_decay);
                adamw_elem(wi.y, gi.y, mi.y, vi.y, tlr, b1, b2, eps, ds.bc1_inv, ds.bc2_inv, ds.weight_decay);
                adamw_elem(wi.z, gi.z, mi.z, vi.z, tlr, b1, b2, eps, ds.bc1_inv, ds.bc2_inv, ds.weight_decay);
                adamw_elem(wi.w, gi.w, mi.w, vi.w, tlr, b1, b2, eps, ds.bc1_inv, ds.bc2_inv, ds.weight_decay);
                if (ds.has_clamp) {
                    wi.x = fminf(fmaxf(wi.x, ds.clamp_lo), ds.clamp_hi);
                    wi.y = fminf(fmaxf(wi.y, ds.clamp_lo), ds.clamp_hi);
                    wi.z = fminf(fmaxf(wi.z, ds.clamp_lo), ds.clamp_hi);
                    wi.w = fminf(fmaxf(wi.w, ds.clamp_lo), ds.clamp_hi);
                }
                w4[i] = wi; m4[i] = mi; v4[i] = vi;
            }
        } else {
            for (int i = threadIdx.x; i < len; i += blockDim.x) {
                const long long e = s0 + i;
                float wi = w[e], mi = m[e], vi = v[e];
                adamw_elem(wi, g[e] * gs, mi, vi, tlr, b1, b2, eps, ds.bc1_inv, ds.bc2_inv,
                           ds.weight_decay);
                if (ds.has_clamp) wi = fminf(fmaxf(wi, ds.clamp_lo), ds.clamp_hi);
                w[e] = wi; m[e] = mi; v[e] = vi;
            }
        }
    }
}

// Sum of squares of a flat arena → one float (two-stage, deterministic), then
// norm and clip scale. partial must hold >= gridDim.x floats.
__global__ void __launch_bounds__(AW_THREADS) arena_sumsq_kernel(const float* __restrict__ g,
                                                                 long long n,
                                                                 float* __restrict__ partial)
{
    __shared__ float red[32];
    float s = 0.0f;
    const long long n4 = n >> 2;
    const float4* g4 = reinterpret_cast<const float4*>(g);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const float4 x = g4[i];
        s += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        s += g[i] * g[i];
    const float tot = block_sum(s, red);
    if (threadIdx.x == 0) partial[blockIdx.x] = tot;
}

static int grid_for(long long work_items, int per_cta)
{
    long long need = (work_items + per_cta - 1) / per_cta;
    const long long cap = 148LL * 8;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

}  // namespace nlh

using namespace nlh;

extern "C" {

uint32_t adamw_update_cuda(float* w, const float* g, float* m, float* v, int32_t n, float lr,
                           float beta1, float beta2, float eps, float bc1_inv, float bc2_inv,
                           float weight_decay)
{
    if (n <= 0) return (uint32_t)cudaSuccess;
    cudaStream_t st = current_stream();
    const bool aligned = (((uintptr_t)w | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0;
    long long done = 0;
    if (aligned && n >= 4) {
        const long long n4 = n >> 2;
        adamw_vec4_kernel<<<grid_for(n4, AW_THREADS), AW_THREADS, 0, st>>>(
            (float4*)w, (const float4*)g, (float4*)m, (float4*)v, n4, lr, beta1, beta2, eps,
            bc1_inv, bc2_inv, weight_decay);
        done = n4 << 2;
    }
    if (done < n) {
        adamw_scalar_kernel<<<grid_for(n - done, AW_THREADS), AW_THREADS, 0, st>>>(
            w, g, m, v, done, n, lr, beta1, beta2, eps, bc1_inv, bc2_inv, weight_decay);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) record_status(NLH_ERR_CUDA, "adamw_update_cuda", cudaGetErrorString(e));
    return (uint32_t)e;
}

uint32_t grad_norm_sq_cuda(const float* g, float* partial_sums, int32_t n, int32_t* out_num_blocks)
{
    const long long nb = ((long long)n + 255) / 256;
    if (out_num_blocks) *out_num_blocks = (int32_t)nb;
    if (n <= 0) return (uint32_t)cudaSuccess;
    partial256_kernel<false><<<grid_for(nb, AW_THREADS / 32), AW_THREADS, 0, current_stream()>>>(
        g, nullptr, partial_sums, n, nb);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) record_status(NLH_ERR_CUDA, "grad_norm_sq_cuda", cudaGetErrorString(e));
    return (uint32_t)e;
}

uint32_t dot_product_partial_f32_cuda(const float* a, const float* b, float* partial_sums,
                                      int32_t n, int32_t* out_num_blocks)
{
    const long long nb = ((long long)n + 255) / 256;
    if (out_num_blocks) *out_num_blocks = (int32_t)nb;
    if (n <= 0) return (uint32_t)cudaSuccess;
    partial256_kernel<true><<<grid_for(nb, AW_THREADS / 32), AW_THREADS, 0, current_stream()>>>(
        a, b, partial_sums, n, nb);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        record_status(NLH_ERR_CUDA, "dot_product_partial_f32_cuda", cudaGetErrorString(e));
    return (uint32_t)e;
}

uint32_t grad_scale_cuda(float* g, float scale, int32_t n)
{
    if (n <= 0) return (uint32_t)cudaSuccess;
    scale_kernel<<<grid_for(n, AW_THREADS * 4), AW_THREADS, 0, current_stream()>>>(g, nullptr,
                                                                                   scale, n);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) record_status(NLH_ERR_CUDA, "grad_scale_cuda", cudaGetErrorString(e));
    return (uint32_t)e;
}

uint32_t reduce_partials_clip_cuda(const float* partial_sums, int32_t total_partials,
                                   float max_grad_norm, float* out_norm, float* out_scale)
{
    reduce_partials_clip_kernel<<<1, AW_THREADS, 0, current_stream()>>>(
        partial_sums, total_partials, max_grad_norm, out_norm, out_scale);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        record_status(NLH_ERR_CUDA, "reduce_partials_clip_cuda", cudaGetErrorString(e));
    return (uint32_t)e;
}

uint32_t grad_scale_conditional_cuda(float* g, const float* scale_ptr, int32_t n)
{
    if (n <= 0) return (uint32_t)cudaSuccess;
    scale_kernel<<<grid_for(n, AW_THREADS * 4), AW_THREADS, 0, current_stream()>>>(g, scale_ptr,
                                                                                   1.0f, n);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        record_status(NLH_ERR_CUDA, "grad_scale_conditional_cuda", cudaGetErrorString(e));
    return (uint32_t)e;
}

int32_t nlh_arena_grad_norm_clip(const float* g, int64_t n, float max_grad_norm, float* partial,
                                 int32_t partial_capacity, float* out_norm, float* out_scale)
{
    if (n < 0 || partial == nullptr || partial_capacity < 1) return NLH_ERR_INVALID_ARG;
    if ((((uintptr_t)g) & 15) != 0) return NLH_ERR_INVALID_ARG;
    int grid = grid_for(n >> 2, AW_THREADS * 4);
    if (grid > partial_capacity) grid = partial_capacity;
    cudaStream_t st = current_stream();
    arena_sumsq_kernel<<<grid, AW_THREADS, 0, st>>>(g, n, partial);
    reduce_partials_clip_kernel<<<1, AW_THREADS, 0, st>>>(partial, grid, max_grad_norm, out_norm,
                                                          out_scale);
    return check_launch("nlh_arena_grad_norm_clip") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_adamw_multi_tensor(float* w, const float* g, float* m, float* v,
                               const nlh_adamw_tensor_desc* descs_dev, const int32_t* chunk_tensor_dev,
                               const int64_t* chunk_start_dev, const int32_t* chunk_len_dev,
                               int32_t n_chunks, const float* grad_scale_ptr, float lr, float beta1,
                               float beta2, float eps)
{
    if (n_chunks <= 0) return NLH_OK;
    if (!w || !g || !m || !v || !descs_dev || !chunk_tensor_dev || !chunk_start_dev || !chunk_len_dev)
        return NLH_ERR_INVALID_ARG;
    int grid = n_chunks < 148 * 8 ? n_chunks : 148 * 8;
    adamw_multi_kernel<<<grid, AW_THREADS, 0, current_stream()>>>(
        w, g, m, v, descs_dev, chunk_tensor_dev, (const long long*)chunk_start_dev, chunk_len_dev,
        n_chunks, grad_scale_ptr, lr, beta1, beta2, eps);
    return check_launch("nlh_adamw_multi_tensor") ? NLH_OK : NLH_ERR_CUDA;
}

}  // extern "C"
