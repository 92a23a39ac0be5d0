// Sliding-window attention (with optional persistent prefix) forward and
// backward for sm_100a: band-limited flash attention. bf16 operands, fp32
// accumulation on the tensor cores, online softmax; the [B,H,S,n_p+W] weights
// tensor of the reference is never needed by the math (the backward
// recomputes probabilities from the per-row log-sum-exp) and is written only
// when the drop-in entry is given a non-NULL attn_weights pointer.
//
// Mask (core/kernels/swa_forward.cu:48-60): key kp is visible to query qp iff
//   kp <= qp  and  (kp < n_persistent  or  kp >= qp + 1 - window).
//
// Tiling: 64 queries x 64 keys per step, 4 warps, each warp owns 16 rows of
// the tile; only key tiles that intersect the band (or the prefix) are
// visited. Backward is split in a dK/dV kernel (CTA per key tile, loops over
// the query tiles that see it) and a dQ kernel (CTA per query tile), so no
// fp32 atomics are needed (the reference uses atomicAdd on dK/dV:
// core/kernels/swa_backward.cu:100-160).
#include <cuda_bf16.h>

#include "nlh_common.cuh"
#include "swa_tc_bwd.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {

constexpr int SWA_BM = 64;
constexpr int SWA_BN = 64;
constexpr int SWA_THREADS = 128;
constexpr int SWA_PAD = 8;   // bf16 elements of row padding (16 B): conflict-free ldmatrix

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void cp16(void* smem_dst, const void* gsrc)
{
    unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* smem_ptr)
{
    unsigned s = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned (&r)[4], const void* smem_ptr)
{
    unsigned s = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

__device__ __forceinline__ bool swa_visible(int qp, int kp, int window, int n_p)
{
    return kp <= qp && (kp < n_p || kp >= qp + 1 - window);
}
// Does key tile kt (64 keys) hold any key visible to some query of [q_lo, q_hi]?
__device__ __forceinline__ bool swa_tile_needed(int kt, int q_lo, int q_hi, int window, int n_p)
{
    const int k_lo = kt * SWA_BN, k_hi = k_lo + SWA_BN - 1;
    if (k_lo > q_hi) return false;
    if (k_lo < n_p) return true;             // prefix keys (causality is checked per element)
    return k_hi >= q_lo + 1 - window;        // band of the earliest query reaches this tile
}

// Async copy of a [rows x HD] bf16 tile (rows >= n_valid are zero-filled) into padded smem.
template <int HD>
__device__ __forceinline__ void load_tile_bf16(bf16* dst, const bf16* __restrict__ src, size_t row_stride,
                                               int n_valid)
{
    constexpr int LD = HD + SWA_PAD;
    constexpr int VPR = HD / 8;   // 16-byte vectors per row
    for (int i = threadIdx.x; i < SWA_BM * VPR; i += SWA_THREADS) {
        const int row = i / VPR, vec = i - row * VPR;
        bf16* d = dst + row * LD + vec * 8;
        if (row < n_valid) cp16(d, src + (size_t)row * row_stride + vec * 8);
        else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
}
// Synchronous copy of a [rows x HD] fp32 tile converted to bf16.
template <int HD>
__device__ __forceinline__ void load_tile_f32_as_bf16(bf16* dst, const float* __restrict__ src,
                                                      size_t row_stride, int n_valid)
{
    constexpr int LD = HD + SWA_PAD;
    constexpr int VPR = HD / 8;
    for (int i = threadIdx.x; i < SWA_BM * VPR; i += SWA_THREADS) {
        const int row = i / VPR, vec = i - row * VPR;
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (row < n_valid) {
            const float4 a = *reinterpret_cast<const float4*>(src + (size_t)row * row_stride + vec * 8);
            const float4 b = *reinterpret_cast<const float4*>(src + (size_t)row * row_stride + vec * 8 + 4);
            o.x = pack_bf16(a.x, a.y); o.y = pack_bf16(a.z, a.w);
            o.z = pack_bf16(b.x, b.y); o.w = pack_bf16(b.z, b.w);
        }
        *reinterpret_cast<uint4*>(dst + row * LD + vec * 8) = o;
    }
}

// d_out tile in either storage type
template <int HD>
__device__ __forceinline__ void load_tile_do(bf16* dst, const float* src, size_t row_stride, int n_valid)
{
    load_tile_f32_as_bf16<HD>(dst, src, row_stride, n_valid);
}
template <int HD>
__device__ __forceinline__ void load_tile_do(bf16* dst, const bf16* src, size_t row_stride, int n_valid)
{
    load_tile_bf16<HD>(dst, src, row_stride, n_valid);
}
__device__ __forceinline__ float do_as_float(float x) { return x; }
__device__ __forceinline__ float do_as_float(bf16 x) { return __bfloat162float(x); }
// two adjacent gradient elements, in either storage type
template <bool ACCUM>
__device__ __forceinline__ void store_grad2(float* p, float a, float b)
{
    float2 o = make_float2(a, b);
    if (ACCUM) { const float2 old = *reinterpret_cast<float2*>(p); o.x += old.x; o.y += old.y; }
    *reinterpret_cast<float2*>(p) = o;
}
template <bool ACCUM>
__device__ __forceinline__ void store_grad2(bf16* p, float a, float b)
{
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);   // packed gradients are never accumulated
}

// acc[nt][4] (16 x 64, fp32) = A(16 x HD, rows a_row0.. of As) * B^T, with B
// stored [64 rows(n)][HD(k)] (row-major n x k): used for Q K^T, K Q^T, dO V^T, V dO^T.
template <int HD>
__device__ __forceinline__ void gemm_nt_16x64(float (&acc)[8][4], const bf16* As, int a_row0, const bf16* Bs)
{
    constexpr int LD = HD + SWA_PAD;
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
        unsigned a[4];
        ldsm_x4(a, As + (a_row0 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < 4; np++) {
            unsigned b[4];
            ldsm_x4(b, Bs + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
            mma16816(acc[2 * np], a, b[0], b[1]);
            mma16816(acc[2 * np + 1], a, b[2], b[3]);
        }
    }
}
// out[HD/8][4] (16 x HD) += P(16 x 64, register A-fragments pa[4][4]) * B, with B
// stored [64 rows(k)][HD(n)] (row-major k x n): used for P V, P^T dO, dS K, dS^T Q.
template <int HD>
__device__ __forceinline__ void gemm_nn_16xHD(float (&out)[HD / 8][4], const unsigned (&pa)[4][4], const bf16* Bs)
{
    constexpr int LD = HD + SWA_PAD;
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int ks = 0; ks < 4; ks++) {
#pragma unroll
        for (int np = 0; np < HD / 16; np++) {
            unsigned b[4];
            ldsm_x4_t(b, Bs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + np * 16 + (lane >> 4) * 8);
            mma16816(out[2 * np], pa[ks], b[0], b[1]);
            mma16816(out[2 * np + 1], pa[ks], b[2], b[3]);
        }
    }
}
// C-fragment tile (16 x 64 fp32) -> A fragments (bf16) for the next MMA.
__device__ __forceinline__ void c_to_a(unsigned (&pa)[4][4], const float (&c)[8][4])
{
#pragma unroll
    for (int ks = 0; ks < 4; ks++) {
        pa[ks][0] = pack_bf16(c[2 * ks][0], c[2 * ks][1]);
        pa[ks][1] = pack_bf16(c[2 * ks][2], c[2 * ks][3]);
        pa[ks][2] = pack_bf16(c[2 * ks + 1][0], c[2 * ks + 1][1]);
        pa[ks][3] = pack_bf16(c[2 * ks + 1][2], c[2 * ks + 1][3]);
    }
}

// ───────────────────────────── forward ────────────────────────────────────
template <int HD>
__global__ void __launch_bounds__(SWA_THREADS) swa_fwd_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
    bf16* __restrict__ out, float* __restrict__ lse, int S, int H, int window, int n_p, float scale,
    int rs_in, int rs_o)
{
    constexpr int LD = HD + SWA_PAD;
    extern __shared__ __align__(16) unsigned char smraw[];
    bf16* Qs = reinterpret_cast<bf16*>(smraw);
    bf16* Ks = Qs + SWA_BM * LD;            // [2][64][LD]
    bf16* Vs = Ks + 2 * SWA_BN * LD;        // [2][64][LD]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int qt = (gridDim.x - 1) - blockIdx.x;   // long tiles first
    const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
    const size_t rs = (size_t)rs_in;               // row stride of q, k, v (elements)
    const bf16* qb = q + (size_t)b * S * rs + (size_t)h * HD;
    const bf16* kb = k + (size_t)b * S * rs + (size_t)h * HD;
    const bf16* vb = v + (size_t)b * S * rs + (size_t)h * HD;
    bf16* ob = out + (size_t)b * S * rs_o + (size_t)h * HD;
    const int q0 = qt * SWA_BM;
    const int q_hi = min(q0 + SWA_BM - 1, S - 1);
    const float sl2 = scale * 1.4426950408889634f;

    load_tile_bf16<HD>(Qs, qb + (size_t)q0 * rs, rs, min(SWA_BM, S - q0));
    int kt = -1;
    const int kt_last = q_hi / SWA_BN;
    auto next_tile = [&](int cur) {
        for (int t = cur + 1; t <= kt_last; t++)
            if (swa_tile_needed(t, q0, q_hi, window, n_p)) return t;
        return -1;
    };
    auto issue = [&](int tile, int buf) {
        const int k0 = tile * SWA_BN;
        load_tile_bf16<HD>(Ks + buf * SWA_BN * LD, kb + (size_t)k0 * rs, rs, min(SWA_BN, S - k0));
        load_tile_bf16<HD>(Vs + buf * SWA_BN * LD, vb + (size_t)k0 * rs, rs, min(SWA_BN, S - k0));
    };
    kt = next_tile(-1);
    if (kt >= 0) issue(kt, 0);
    cp_commit();

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row0 = q0 + warp * 16 + g;   // rows row0 and row0 + 8

    int buf = 0;
    while (kt >= 0) {
        const int nxt = next_tile(kt);
        if (nxt >= 0) issue(nxt, buf ^ 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
        gemm_nt_16x64<HD>(s, Qs, warp * 16, Ks + buf * SWA_BN * LD);
        const int k0 = kt * SWA_BN;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int kp = k0 + nt * 8 + 2 * t4 + (e & 1);
                const int qp = row0 + (e >> 1) * 8;
                const bool ok = kp < S && swa_visible(qp, kp, window, n_p);
                s[nt][e] = ok ? s[nt][e] : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
            }
        }
        float corr[2], mu[2];
#pragma unroll
        for (int r2 = 0; r2 < 2; r2++) {
            mx[r2] = fmaxf(mx[r2], __shfl_xor_sync(0xffffffffu, mx[r2], 1));
            mx[r2] = fmaxf(mx[r2], __shfl_xor_sync(0xffffffffu, mx[r2], 2));
            const float m_new = fmaxf(m_run[r2], mx[r2]);
            mu[r2] = (m_new == -INFINITY) ? 0.f : m_new;
            corr[r2] = exp2f((m_run[r2] - mu[r2]) * sl2);   // m_run = -inf -> 0
            m_run[r2] = m_new;
            l_run[r2] *= corr[r2];
        }
        float ls[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = exp2f((s[nt][e] - mu[e >> 1]) * sl2);
                s[nt][e] = p;
                ls[e >> 1] += p;
            }
        }
        l_run[0] += ls[0]; l_run[1] += ls[1];
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        unsigned pa[4][4];
        c_to_a(pa, s);
        gemm_nn_16xHD<HD>(o, pa, Vs + buf * SWA_BN * LD);
        __syncthreads();   // all warps done with this buffer before it is refilled
        kt = nxt;
        buf ^= 1;
    }
    cp_wait<0>();
#pragma unroll
    for (int r2 = 0; r2 < 2; r2++) {
        l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 1);
        l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 2);
    }
#pragma unroll
    for (int r2 = 0; r2 < 2; r2++) {
        const int qp = row0 + r2 * 8;
        if (qp < S) {
            const float inv = (l_run[r2] > 0.f) ? 1.0f / l_run[r2] : 0.f;
#pragma unroll
            for (int i = 0; i < HD / 8; i++) {
                __nv_bfloat162 w = __floats2bfloat162_rn(o[i][2 * r2] * inv, o[i][2 * r2 + 1] * inv);
                *reinterpret_cast<__nv_bfloat162*>(ob + (size_t)qp * rs_o + i * 8 + 2 * t4) = w;
            }
            if (t4 == 0 && lse != nullptr)
                lse[((size_t)b * H + h) * S + qp] = m_run[r2] * scale + logf(l_run[r2]);
        }
    }
}

// attn_weights[b,h,qp,slot] for the drop-in entry: slot w < n_p is key w, slot
// n_p + w is key local_start + w (core/kernels/swa_forward.cu:134-146).
// One warp per query row, lanes stride over slots.
template <int HD>
__global__ void __launch_bounds__(256) swa_weights_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k, const float* __restrict__ lse,
    bf16* __restrict__ aw, int S, int H, int window, int n_p, int B, float scale)
{
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (long long)B * H * S) return;
    const int qp = (int)(row % S);
    const int h = (int)((row / S) % H);
    const int b = (int)(row / ((long long)S * H));
    const size_t rs = (size_t)H * HD;
    const bf16* qr = q + ((size_t)b * S + qp) * rs + (size_t)h * HD;
    const bf16* kb = k + (size_t)b * S * rs + (size_t)h * HD;
    const int aws = n_p + window;
    bf16* wr = aw + (size_t)row * aws;
    const float l = lse[row];
    const int n_p_att = (qp + 1 < n_p) ? qp + 1 : n_p;
    int local_start = 0, local_len = 0;
    if (qp >= n_p) {
        local_start = (qp + 1 - window > n_p) ? (qp + 1 - window) : n_p;
        local_len = qp + 1 - local_start;
    }
    float qf[HD];
#pragma unroll
    for (int i = 0; i < HD; i++) qf[i] = __bfloat162float(qr[i]);
    for (int w = lane; w < aws; w += 32) {
        int kp = -1;
        if (w < n_p) { if (w < n_p_att) kp = w; }
        else if (w - n_p < local_len) kp = local_start + (w - n_p);
        float val = 0.f;
        if (kp >= 0) {
            const bf16* kr = kb + (size_t)kp * rs;
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < HD; i++) dot += qf[i] * __bfloat162float(kr[i]);
            val = expf(dot * scale - l);
        }
        wr[w] = __float2bfloat16(val);
    }
}

// delta[b,h,q] = sum_d dO[q,d] * O[q,d]
template <int HD, typename TDO>
__global__ void __launch_bounds__(256) swa_delta_kernel(const TDO* __restrict__ d_out,
                                                        const bf16* __restrict__ out,
                                                        float* __restrict__ delta, int S, int H, int B, int rs_o,
                                                        bf16* __restrict__ do16)
{
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (long long)B * H * S) return;
    const int qp = (int)(row % S);
    const int h = (int)((row / S) % H);
    const int b = (int)(row / ((long long)S * H));
    const size_t off = ((size_t)b * S + qp) * rs_o + (size_t)h * HD;
    float s = 0.f;
    // do16 (optional): dense bf16 copy of the upstream gradient for the tensor-core kernels
    const size_t off16 = ((size_t)b * S + qp) * ((size_t)H * HD) + (size_t)h * HD;
    for (int i = lane; i < HD; i += 32) {
        const float g = do_as_float(d_out[off + i]);
        s += g * __bfloat162float(out[off + i]);
        if (do16 != nullptr) do16[off16 + i] = __float2bfloat16(g);
    }
    s = warp_sum(s);
    if (lane == 0) delta[row] = s;
}

// Same pre-pass with 16-byte accesses: HD/8 lanes per (b,h,q) row, 8 elements per lane. Needs
// 16-byte aligned bases and row strides that are multiples of 8 elements.
__device__ __forceinline__ void ld8_do(const bf16* p, float (&x)[8])
{
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; i++) { x[2 * i] = __low2float(h[i]); x[2 * i + 1] = __high2float(h[i]); }
}
__device__ __forceinline__ void ld8_do(const float* p, float (&x)[8])
{
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
template <int HD, typename TDO>
__global__ void __launch_bounds__(256) swa_delta_vec_kernel(const TDO* __restrict__ d_out,
                                                            const bf16* __restrict__ out,
                                                            float* __restrict__ delta, int S, int H, int B, int rs_o,
                                                            bf16* __restrict__ do16)
{
    constexpr int LPR = HD / 8;                      // lanes per row: 4, 8 or 16
    static_assert(LPR >= 1 && LPR <= 32 && (LPR & (LPR - 1)) == 0, "head_dim / 8 must be a power of two <= 32");
    const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long row = gt / LPR;
    const int c = (int)(gt - row * LPR) * 8;
    const bool live = row < (long long)B * H * S;
    float s = 0.f;
    if (live) {
        const int qp = (int)(row % S);
        const int h = (int)((row / S) % H);
        const int b = (int)(row / ((long long)S * H));
        const size_t off = ((size_t)b * S + qp) * rs_o + (size_t)h * HD + c;
        float g[8], o[8];
        ld8_do(d_out + off, g);
        ld8_do(out + off, o);
#pragma unroll
        for (int i = 0; i < 8; i++) s += g[i] * o[i];
        if (do16 != nullptr) {
            uint4 u;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
            for (int i = 0; i < 4; i++) h2[i] = __floats2bfloat162_rn(g[2 * i], g[2 * i + 1]);
            *reinterpret_cast<uint4*>(do16 + ((size_t)b * S + qp) * ((size_t)H * HD) + (size_t)h * HD + c) = u;
        }
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (live && c == 0) delta[row] = s;
}

// ───────────────────────────── backward: dK, dV ───────────────────────────
// CTA = one tile of 64 keys; warp = 16 keys (rows of S^T). Loops over the
// query tiles that can see the key tile.
template <int HD, bool ACCUM, typename TDO, typename TG>
__global__ void __launch_bounds__(SWA_THREADS) swa_bwd_dkv_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
    const TDO* __restrict__ d_out, const float* __restrict__ lse, const float* __restrict__ delta,
    TG* __restrict__ d_k, TG* __restrict__ d_v, int S, int H, int window, int n_p, float scale,
    int rs_in, int rs_o)
{
    constexpr int LD = HD + SWA_PAD;
    extern __shared__ __align__(16) unsigned char smraw[];
    bf16* Ks = reinterpret_cast<bf16*>(smraw);   // [64][LD]
    bf16* Vs = Ks + SWA_BN * LD;
    bf16* Qs = Vs + SWA_BN * LD;                 // [64][LD]
    bf16* dOs = Qs + SWA_BM * LD;                // [64][LD]
    float* lse_s = reinterpret_cast<float*>(dOs + SWA_BM * LD);   // [64]
    float* del_s = lse_s + SWA_BM;                                // [64]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int kt = blockIdx.x;
    const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
    const size_t rs = (size_t)rs_in;                      // row stride of q, k, v and their gradients
    const size_t base = (size_t)b * S * rs + (size_t)h * HD;
    const size_t base_o = (size_t)b * S * rs_o + (size_t)h * HD;   // d_out rows
    const int k0 = kt * SWA_BN;
    const int k_hi = min(k0 + SWA_BN - 1, S - 1);
    const float sl2 = scale * 1.4426950408889634f;

    load_tile_bf16<HD>(Ks, k + base + (size_t)k0 * rs, rs, min(SWA_BN, S - k0));
    load_tile_bf16<HD>(Vs, v + base + (size_t)k0 * rs, rs, min(SWA_BN, S - k0));
    cp_commit();

    float dk[HD / 8][4], dv[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) {
        dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
        dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
    }
    const int krow0 = k0 + warp * 16 + g;   // keys krow0 and krow0 + 8

    // query tiles: from the tile holding k0 up to the last query that sees k_hi
    const int q_last = (k0 < n_p) ? (S - 1) : min(S - 1, k_hi + window - 1);
    const int qt_first = k0 / SWA_BM, qt_last = q_last / SWA_BM;
    for (int qt = qt_first; qt <= qt_last; qt++) {
        const int q0 = qt * SWA_BM;
        const int nq = min(SWA_BM, S - q0);
        __syncthreads();   // previous iteration's readers are done with Qs/dOs/lse_s
        load_tile_bf16<HD>(Qs, q + base + (size_t)q0 * rs, rs, nq);
        load_tile_do<HD>(dOs, d_out + base_o + (size_t)q0 * rs_o, (size_t)rs_o, nq);
        cp_commit();
        if (threadIdx.x < SWA_BM) {
            const int qp = q0 + threadIdx.x;
            lse_s[threadIdx.x] = (qp < S) ? lse[((size_t)b * H + h) * S + qp] : 0.f;
            del_s[threadIdx.x] = (qp < S) ? delta[((size_t)b * H + h) * S + qp] : 0.f;
        }
        cp_wait<0>();
        __syncthreads();
        // S^T = K Q^T  (rows: keys of this warp, cols: 64 queries)
        float st[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) { st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f; }
        gemm_nt_16x64<HD>(st, Ks, warp * 16, Qs);
        // dP^T = V dO^T
        float dp[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) { dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f; }
        gemm_nt_16x64<HD>(dp, Vs, warp * 16, dOs);
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int ql = nt * 8 + 2 * t4 + (e & 1);
                const int qp = q0 + ql;
                const int kp = krow0 + (e >> 1) * 8;
                const bool ok = qp < S && kp < S && swa_visible(qp, kp, window, n_p);
                const float p = ok ? exp2f(st[nt][e] * sl2 - lse_s[ql] * 1.4426950408889634f) : 0.f;
                st[nt][e] = p;                                      // P^T
                dp[nt][e] = p * (dp[nt][e] - del_s[ql]) * scale;    // dS^T (already scaled)
            }
        }
        unsigned pa[4][4];
        c_to_a(pa, st);
        gemm_nn_16xHD<HD>(dv, pa, dOs);    // dV += P^T dO
        c_to_a(pa, dp);
        gemm_nn_16xHD<HD>(dk, pa, Qs);     // dK += dS^T Q
    }
#pragma unroll
    for (int r2 = 0; r2 < 2; r2++) {
        const int kp = krow0 + r2 * 8;
        if (kp < S) {
            TG* dkr = d_k + base + (size_t)kp * rs;
            TG* dvr = d_v + base + (size_t)kp * rs;
#pragma unroll
            for (int i = 0; i < HD / 8; i++) {
                const int c = i * 8 + 2 * t4;
                store_grad2<ACCUM>(dkr + c, dk[i][2 * r2], dk[i][2 * r2 + 1]);
                store_grad2<ACCUM>(dvr + c, dv[i][2 * r2], dv[i][2 * r2 + 1]);
            }
        }
    }
}

// ───────────────────────────── backward: dQ ───────────────────────────────
template <int HD, typename TDO, typename TG>
__global__ void __launch_bounds__(SWA_THREADS) swa_bwd_dq_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
    const TDO* __restrict__ d_out, const float* __restrict__ lse, const float* __restrict__ delta,
    TG* __restrict__ d_q, int S, int H, int window, int n_p, float scale, int rs_in, int rs_o)
{
    constexpr int LD = HD + SWA_PAD;
    extern __shared__ __align__(16) unsigned char smraw[];
    bf16* Qs = reinterpret_cast<bf16*>(smraw);
    bf16* dOs = Qs + SWA_BM * LD;
    bf16* Ks = dOs + SWA_BM * LD;            // [2][64][LD]
    bf16* Vs = Ks + 2 * SWA_BN * LD;         // [2][64][LD]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int qt = (gridDim.x - 1) - blockIdx.x;
    const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
    const size_t rs = (size_t)rs_in;
    const size_t base = (size_t)b * S * rs + (size_t)h * HD;
    const size_t base_o = (size_t)b * S * rs_o + (size_t)h * HD;
    const int q0 = qt * SWA_BM;
    const int q_hi = min(q0 + SWA_BM - 1, S - 1);
    const float sl2 = scale * 1.4426950408889634f;
    const int nq = min(SWA_BM, S - q0);

    load_tile_bf16<HD>(Qs, q + base + (size_t)q0 * rs, rs, nq);
    load_tile_do<HD>(dOs, d_out + base_o + (size_t)q0 * rs_o, (size_t)rs_o, nq);
    const int kt_last = q_hi / SWA_BN;
    auto next_tile = [&](int cur) {
        for (int t = cur + 1; t <= kt_last; t++)
            if (swa_tile_needed(t, q0, q_hi, window, n_p)) return t;
        return -1;
    };
    auto issue = [&](int tile, int buf) {
        const int k0 = tile * SWA_BN;
        load_tile_bf16<HD>(Ks + buf * SWA_BN * LD, k + base + (size_t)k0 * rs, rs, min(SWA_BN, S - k0));
        load_tile_bf16<HD>(Vs + buf * SWA_BN * LD, v + base + (size_t)k0 * rs, rs, min(SWA_BN, S - k0));
    };
    int kt = next_tile(-1);
    if (kt >= 0) issue(kt, 0);
    cp_commit();

    const int row0 = q0 + warp * 16 + g;
    float lse_r[2], del_r[2];
#pragma unroll
    for (int r2 = 0; r2 < 2; r2++) {
        const int qp = row0 + r2 * 8;
        lse_r[r2] = (qp < S) ? lse[((size_t)b * H + h) * S + qp] * 1.4426950408889634f : 0.f;
        del_r[r2] = (qp < S) ? delta[((size_t)b * H + h) * S + qp] : 0.f;
    }
    float dq[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) { dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f; }

    int buf = 0;
    while (kt >= 0) {
        const int nxt = next_tile(kt);
        if (nxt >= 0) issue(nxt, buf ^ 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        float s[8][4], dp[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
        }
        gemm_nt_16x64<HD>(s, Qs, warp * 16, Ks + buf * SWA_BN * LD);     // S = Q K^T
        gemm_nt_16x64<HD>(dp, dOs, warp * 16, Vs + buf * SWA_BN * LD);   // dP = dO V^T
        const int k0 = kt * SWA_BN;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int kp = k0 + nt * 8 + 2 * t4 + (e & 1);
                const int qp = row0 + (e >> 1) * 8;
                const bool ok = qp < S && kp < S && swa_visible(qp, kp, window, n_p);
                const float p = ok ? exp2f(s[nt][e] * sl2 - lse_r[e >> 1]) : 0.f;
                dp[nt][e] = p * (dp[nt][e] - del_r[e >> 1]) * scale;
            }
        }
        unsigned pa[4][4];
        c_to_a(pa, dp);
        gemm_nn_16xHD<HD>(dq, pa, Ks + buf * SWA_BN * LD);   // dQ += dS K
        __syncthreads();
        kt = nxt;
        buf ^= 1;
    }
    cp_wait<0>();
#pragma unroll
    for (int r2 = 0; r2 < 2; r2++) {
        const int qp = row0 + r2 * 8;
        if (qp < S) {
            TG* dqr = d_q + base + (size_t)qp * rs;
#pragma unroll
            for (int i = 0; i < HD / 8; i++)
                store_grad2<false>(dqr + i * 8 + 2 * t4, dq[i][2 * r2], dq[i][2 * r2 + 1]);
        }
    }
}

// ───────────────────────────── host side ──────────────────────────────────
// nlh_set_option(NLH_OPT_SWA_TCGEN05, 0) switches the head_dim-64 forward
template <int HD>
static size_t swa_fwd_smem() { return (size_t)(SWA_BM + 4 * SWA_BN) * (HD + SWA_PAD) * sizeof(bf16); }
template <int HD>
static size_t swa_dkv_smem() { return (size_t)(2 * SWA_BN + 2 * SWA_BM) * (HD + SWA_PAD) * sizeof(bf16) + 2 * SWA_BM * sizeof(float); }
template <int HD>
static size_t swa_dq_smem() { return (size_t)(2 * SWA_BM + 4 * SWA_BN) * (HD + SWA_PAD) * sizeof(bf16); }

static int swa_check(const char* where, int S, int H, int hd, int W, int B, int n_p)
{
    if (S <= 0 || H <= 0 || B < 0 || W <= 0 || n_p < 0) {
        record_status(NLH_ERR_INVALID_ARG, where, "seq_len, num_heads, window_size must be > 0; batch, n_persistent >= 0");
        return NLH_ERR_INVALID_ARG;
    }
    if (!(hd == 16 || hd == 32 || hd == 64 || hd == 128)) {
        record_status(NLH_ERR_UNSUPPORTED, where, "head_dim must be 16, 32, 64 or 128");
        return NLH_ERR_UNSUPPORTED;
    }
    return NLH_OK;
}

// Tiled TMA descriptor of one of q, k, v as the tcgen05 forward stages it: a 3-D bf16 tensor
// {H*64 head-dim elements, S positions (stride rs elements), B batch elements (stride S*rs)}, box
// {8 elements, rows, 1}. The driver's encoder is reached through cudaGetDriverEntryPoint (no link
// against libcuda). Returns false when the encoder is not available or rejects the shape; the
// caller then stages with cp.async.
static int g_swa_fwd_staging = -1;     // staging of the last tcgen05 forward launch: 1 TMA, 0 cp.async
typedef CUresult (*TmaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TmaEncodeFn tma_encode_fn()
{
    static TmaEncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess ||
            qr != cudaDriverEntryPointSuccess)
            p = nullptr;
        (void)cudaGetLastError();
        return (TmaEncodeFn)p;
    }();
    return fn;
}
static bool swa_tile_map(CUtensorMap* m, const bf16* base, int S, int H, int B, int rs, int rows)
{
    TmaEncodeFn enc = tma_encode_fn();
    if (enc == nullptr || (rs % 8) != 0 || (((uintptr_t)base) & 15) != 0) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)H * 64, (cuuint64_t)S, (cuuint64_t)B};
    const cuuint64_t strides[2] = {(cuuint64_t)rs * 2, (cuuint64_t)S * rs * 2};     // bytes, dims 1 and 2
    const cuuint32_t box[3] = {8, (cuuint32_t)rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<bf16*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int HD>
static int swa_forward_impl(const bf16* q, const bf16* k, const bf16* v, bf16* out, float* lse,
                            bf16* aw, int S, int H, int W, int B, int n_p, int rs_in = 0, int rs_o = 0)
{
    cudaStream_t st = current_stream();
    const float scale = 1.0f / sqrtf((float)HD);
    if (rs_in == 0) rs_in = H * HD;     // dense [B, S, H*hd] rows unless the caller packs q|k|v
    if (rs_o == 0) rs_o = H * HD;
    const bool aligned = ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) == 0);
    if (HD == 64 && option_value(NLH_OPT_SWA_TCGEN05) && aligned) {
        // tcgen05 / TMEM kernel: 128 query rows per CTA; operand tiles staged by TMA when the
        // descriptors can be made, else by cp.async
        dim3 grid((S + tc::BM - 1) / tc::BM, B * H);
        CUtensorMap mq, mk, mv;
        memset(&mq, 0, sizeof(mq)); memset(&mk, 0, sizeof(mk)); memset(&mv, 0, sizeof(mv));
        const bool tma = option_value(NLH_OPT_SWA_TMA) && swa_tile_map(&mq, q, S, H, B, rs_in, tc::BM) &&
                         swa_tile_map(&mk, k, S, H, B, rs_in, tc::BN) && swa_tile_map(&mv, v, S, H, B, rs_in, tc::BN);
        g_swa_fwd_staging = tma ? 1 : 0;
        if (tma) {
            cudaFuncSetAttribute(tc::swa_fwd_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
            tc::swa_fwd_tc_kernel<true><<<grid, tc::THREADS, tc::SMEM_BYTES, st>>>(q, k, v, out, lse, S, H, W, n_p, scale, rs_in, rs_o, mq, mk, mv);
        } else {
            cudaFuncSetAttribute(tc::swa_fwd_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
            tc::swa_fwd_tc_kernel<false><<<grid, tc::THREADS, tc::SMEM_BYTES, st>>>(q, k, v, out, lse, S, H, W, n_p, scale, rs_in, rs_o, mq, mk, mv);
        }
        if (!check_launch("swa_fwd_tc_kernel")) return NLH_ERR_CUDA;
    } else {
        const size_t smem = swa_fwd_smem<HD>();
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(swa_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        dim3 grid((S + SWA_BM - 1) / SWA_BM, B * H);
        swa_fwd_kernel<HD><<<grid, SWA_THREADS, smem, st>>>(q, k, v, out, lse, S, H, W, n_p, scale, rs_in, rs_o);
        if (!check_launch("swa_fwd_kernel")) return NLH_ERR_CUDA;
    }
    if (aw != nullptr) {
        const long long rows = (long long)B * H * S;
        swa_weights_kernel<HD><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(q, k, lse, aw, S, H, W, n_p, B, scale);
        if (!check_launch("swa_weights_kernel")) return NLH_ERR_CUDA;
    }
    return NLH_OK;
}

// do16_scratch: B*S*H*HD bf16 of scratch for the converted upstream gradient when TDO is float
// (NULL: the tensor-core kernels are not used for an fp32 upstream gradient).
template <int HD, typename TDO, typename TG>
static int swa_backward_impl(const bf16* q, const bf16* k, const bf16* v, const bf16* out,
                             const float* lse, const TDO* d_out, float* delta, TG* d_q,
                             TG* d_k, TG* d_v, int S, int H, int W, int B, int n_p, bool accum,
                             int rs_in = 0, int rs_o = 0, bf16* do16_scratch = nullptr)
{
    cudaStream_t st = current_stream();
    const float scale = 1.0f / sqrtf((float)HD);
    if (rs_in == 0) rs_in = H * HD;
    if (rs_o == 0) rs_o = H * HD;
    const long long rows = (long long)B * H * S;
    constexpr bool DO_IS_BF16 = sizeof(TDO) == 2;
    const bool aligned = ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)d_out | (uintptr_t)d_q |
                            (uintptr_t)d_k | (uintptr_t)d_v | (uintptr_t)do16_scratch) & 15) == 0) &&
                         (rs_in % 8 == 0) && (rs_o % 8 == 0);
    const bool use_tc = HD == 64 && option_value(NLH_OPT_SWA_TCGEN05) && aligned && (DO_IS_BF16 || do16_scratch != nullptr);
    bf16* do16 = (use_tc && !DO_IS_BF16) ? do16_scratch : nullptr;
    const bool delta_vec = HD % 8 == 0 && (rs_o % 8 == 0) && ((H * HD) % 8 == 0) &&
                           ((((uintptr_t)d_out | (uintptr_t)out | (uintptr_t)do16) & 15) == 0);
    if (delta_vec) {
        const long long lanes = rows * (HD / 8);
        swa_delta_vec_kernel<HD, TDO><<<(unsigned)((lanes + 255) / 256), 256, 0, st>>>(d_out, out, delta, S, H, B, rs_o, do16);
    } else {
        swa_delta_kernel<HD, TDO><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(d_out, out, delta, S, H, B, rs_o, do16);
    }
    if (!check_launch("swa_delta_kernel")) return NLH_ERR_CUDA;
    if (use_tc) {
        // tcgen05 / TMEM kernels: 128 key rows (dK, dV) and 128 query rows (dQ) per CTA
        const bf16* g16 = DO_IS_BF16 ? reinterpret_cast<const bf16*>(d_out) : do16;
        const int rs16 = DO_IS_BF16 ? rs_o : H * HD;
        dim3 grid((S + tc::BM - 1) / tc::BM, B * H);
        if (accum) {
            cudaFuncSetAttribute(tc::swa_bwd_dkv_tc_kernel<TG, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::KV_SMEM_BYTES);
            tc::swa_bwd_dkv_tc_kernel<TG, true><<<grid, tc::BTHREADS, tc::KV_SMEM_BYTES, st>>>(
                q, k, v, g16, lse, delta, d_k, d_v, S, H, W, n_p, scale, rs_in, rs16);
        } else {
            cudaFuncSetAttribute(tc::swa_bwd_dkv_tc_kernel<TG, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::KV_SMEM_BYTES);
            tc::swa_bwd_dkv_tc_kernel<TG, false><<<grid, tc::BTHREADS, tc::KV_SMEM_BYTES, st>>>(
                q, k, v, g16, lse, delta, d_k, d_v, S, H, W, n_p, scale, rs_in, rs16);
        }
        if (!check_launch("swa_bwd_dkv_tc_kernel")) return NLH_ERR_CUDA;
        cudaFuncSetAttribute(tc::swa_bwd_dq_tc_kernel<TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::DQ_SMEM_BYTES);
        tc::swa_bwd_dq_tc_kernel<TG><<<grid, tc::BTHREADS, tc::DQ_SMEM_BYTES, st>>>(
            q, k, v, g16, lse, delta, d_q, S, H, W, n_p, scale, rs_in, rs16);
        return check_launch("swa_bwd_dq_tc_kernel") ? NLH_OK : NLH_ERR_CUDA;
    }
    {
        const size_t smem = swa_dkv_smem<HD>();
        dim3 grid((S + SWA_BN - 1) / SWA_BN, B * H);
        if (accum) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(swa_bwd_dkv_kernel<HD, true, TDO, TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            swa_bwd_dkv_kernel<HD, true, TDO, TG><<<grid, SWA_THREADS, smem, st>>>(q, k, v, d_out, lse, delta, d_k, d_v, S, H, W, n_p, scale, rs_in, rs_o);
        } else {
            if (smem > 48 * 1024) cudaFuncSetAttribute(swa_bwd_dkv_kernel<HD, false, TDO, TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            swa_bwd_dkv_kernel<HD, false, TDO, TG><<<grid, SWA_THREADS, smem, st>>>(q, k, v, d_out, lse, delta, d_k, d_v, S, H, W, n_p, scale, rs_in, rs_o);
        }
        if (!check_launch("swa_bwd_dkv_kernel")) return NLH_ERR_CUDA;
    }
    {
        const size_t smem = swa_dq_smem<HD>();
        if (smem > 48 * 1024) cudaFuncSetAttribute(swa_bwd_dq_kernel<HD, TDO, TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        dim3 grid((S + SWA_BM - 1) / SWA_BM, B * H);
        swa_bwd_dq_kernel<HD, TDO, TG><<<grid, SWA_THREADS, smem, st>>>(q, k, v, d_out, lse, delta, d_q, S, H, W, n_p, scale, rs_in, rs_o);
        if (!check_launch("swa_bwd_dq_kernel")) return NLH_ERR_CUDA;
    }
    return NLH_OK;
}

#define SWA_DISPATCH_HD(hd, ...)                         \
    switch (hd) {                                        \
        case 16: { constexpr int HD_ = 16; __VA_ARGS__; } break;   \
        case 32: { constexpr int HD_ = 32; __VA_ARGS__; } break;   \
        case 64: { constexpr int HD_ = 64; __VA_ARGS__; } break;   \
        default: { constexpr int HD_ = 128; __VA_ARGS__; } break;  \
    }

}  // namespace nlh

using namespace nlh;

extern "C" {

int32_t nlh_swa_tc_timeout_flag(void)
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_swa_tc_timeout, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

int32_t nlh_swa_forward_staging(void) { return g_swa_fwd_staging; }

int32_t nlh_swa_forward(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out,
    float* lse, int32_t seq_len, int32_t num_heads, int32_t head_dim, int32_t window_size,
    int32_t batch_size, int32_t n_persistent)
{
    int rc = swa_check("nlh_swa_forward", seq_len, num_heads, head_dim, window_size, batch_size, n_persistent);
    if (rc != NLH_OK || batch_size == 0) return rc;
    SWA_DISPATCH_HD(head_dim, rc = swa_forward_impl<HD_>((const bf16*)q, (const bf16*)k, (const bf16*)v,
        (bf16*)out, lse, nullptr, seq_len, num_heads, window_size, batch_size, n_persistent));
    return rc;
}

int32_t nlh_swa_backward(const uint16_t* q, const uint16_t* k, const uint16_t* v,
    const uint16_t* out, const float* lse, const float* d_attn_out, float* d_q, float* d_k,
    float* d_v, int32_t seq_len, int32_t num_heads, int32_t head_dim, int32_t window_size,
    int32_t batch_size, int32_t n_persistent)
{
    int rc = swa_check("nlh_swa_backward", seq_len, num_heads, head_dim, window_size, batch_size, n_persistent);
    if (rc != NLH_OK || batch_size == 0) return rc;
    const size_t rows = (size_t)batch_size * num_heads * seq_len;
    const size_t row_bytes = (rows * sizeof(float) + 255) & ~(size_t)255;
    char* ws = (char*)workspace(row_bytes + rows * head_dim * sizeof(bf16));
    if (!ws) return NLH_ERR_WORKSPACE;
    float* delta = (float*)ws;
    bf16* do16 = (bf16*)(ws + row_bytes);       // bf16 copy of the fp32 upstream gradient
    SWA_DISPATCH_HD(head_dim, rc = swa_backward_impl<HD_, float, float>((const bf16*)q, (const bf16*)k, (const bf16*)v,
        (const bf16*)out, lse, d_attn_out, delta, d_q, d_k, d_v, seq_len, num_heads, window_size,
        batch_size, n_persistent, false, 0, 0, do16));
    return rc;
}

int32_t nlh_swa_forward_packed(const uint16_t* qkv, uint16_t* out, float* lse, int32_t seq_len,
    int32_t num_heads, int32_t head_dim, int32_t window_size, int32_t batch_size, int32_t n_persistent)
{
    int rc = swa_check("nlh_swa_forward_packed", seq_len, num_heads, head_dim, window_size, batch_size, n_persistent);
    if (rc != NLH_OK || batch_size == 0) return rc;
    const int dm = num_heads * head_dim;
    const bf16* p = (const bf16*)qkv;
    SWA_DISPATCH_HD(head_dim, rc = swa_forward_impl<HD_>(p, p + dm, p + 2 * dm, (bf16*)out, lse, nullptr,
        seq_len, num_heads, window_size, batch_size, n_persistent, 3 * dm, dm));
    return rc;
}

int32_t nlh_swa_backward_packed(const uint16_t* qkv, const uint16_t* out, const float* lse,
    const uint16_t* d_attn_out, uint16_t* d_qkv, int32_t seq_len, int32_t num_heads, int32_t head_dim,
    int32_t window_size, int32_t batch_size, int32_t n_persistent)
{
    int rc = swa_check("nlh_swa_backward_packed", seq_len, num_heads, head_dim, window_size, batch_size, n_persistent);
    if (rc != NLH_OK || batch_size == 0) return rc;
    const size_t rows = (size_t)batch_size * num_heads * seq_len;
    float* delta = (float*)workspace(rows * sizeof(float));
    if (!delta) return NLH_ERR_WORKSPACE;
    const int dm = num_heads * head_dim;
    const bf16* p = (const bf16*)qkv;
    bf16* g = (bf16*)d_qkv;
    SWA_DISPATCH_HD(head_dim, rc = (swa_backward_impl<HD_, bf16, bf16>(p, p + dm, p + 2 * dm,
        (const bf16*)out, lse, (const bf16*)d_attn_out, delta, g, g + dm, g + 2 * dm, seq_len, num_heads,
        window_size, batch_size, n_persistent, false, 3 * dm, dm)));
    return rc;
}

void swa_forward_f32_cuda(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out,
    uint16_t* attn_weights, int32_t seq_len, int32_t num_heads, int32_t head_dim,
    int32_t window_size, int32_t batch_size, int32_t n_persistent)
{
    int rc = swa_check("swa_forward_f32_cuda", seq_len, num_heads, head_dim, window_size, batch_size, n_persistent);
    if (rc != NLH_OK || batch_size == 0) return;
    const size_t rows = (size_t)batch_size * num_heads * seq_len;
    float* lse = (float*)workspace(rows * sizeof(float));
    if (!lse) return;
    SWA_DISPATCH_HD(head_dim, rc = swa_forward_impl<HD_>((const bf16*)q, (const bf16*)k, (const bf16*)v,
        (bf16*)out, lse, (bf16*)attn_weights, seq_len, num_heads, window_size, batch_size, n_persistent));
}

// The stored weights are a deterministic function of q and k, so the backward
// recomputes out and the log-sum-exp into scratch instead of reading the
// [B,H,S,n_p+W] tensor back from HBM; attn_weights is accepted and not read.
void swa_backward_f32_cuda(const uint16_t* q, const uint16_t* k, const uint16_t* v,
    const uint16_t* attn_weights, const float* d_attn_out, float* d_q, float* d_k, float* d_v,
    int32_t seq_len, int32_t num_heads, int32_t head_dim, int32_t window_size, int32_t batch_size,
    int32_t n_persistent)
{
    (void)attn_weights;
    int rc = swa_check("swa_backward_f32_cuda", seq_len, num_heads, head_dim, window_size, batch_size, n_persistent);
    if (rc != NLH_OK || batch_size == 0) return;
    const size_t rows = (size_t)batch_size * num_heads * seq_len;
    const size_t row_bytes = (rows * sizeof(float) + 255) & ~(size_t)255;
    const size_t out_bytes = ((size_t)batch_size * seq_len * num_heads * head_dim * sizeof(bf16) + 255) & ~(size_t)255;
    char* ws = (char*)workspace(2 * row_bytes + 2 * out_bytes);
    if (!ws) return;
    float* lse = (float*)ws;
    float* delta = (float*)(ws + row_bytes);
    bf16* out = (bf16*)(ws + 2 * row_bytes);
    bf16* do16 = (bf16*)(ws + 2 * row_bytes + out_bytes);
    SWA_DISPATCH_HD(head_dim, rc = swa_forward_impl<HD_>((const bf16*)q, (const bf16*)k, (const bf16*)v,
        out, lse, nullptr, seq_len, num_heads, window_size, batch_size, n_persistent));
    if (rc != NLH_OK) return;
    SWA_DISPATCH_HD(head_dim, rc = swa_backward_impl<HD_, float, float>((const bf16*)q, (const bf16*)k, (const bf16*)v,
        out, lse, d_attn_out, delta, d_q, d_k, d_v, seq_len, num_heads, window_size, batch_size,
        n_persistent, true, 0, 0, do16));
}

}  // extern "C"
