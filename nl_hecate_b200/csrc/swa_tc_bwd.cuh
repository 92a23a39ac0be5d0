// SWA backward on the 5th-generation tensor cores (tcgen05) with TMEM accumulators, head_dim 64.
// Function replaced: swa_backward_kernel, core/kernels/swa_backward.cu:24-162 (one CTA per query,
// stored bf16 weights re-read, fp32 atomicAdd on dK/dV). Here P is recomputed from the log-sum-exp
// of the forward and no atomics are used: two kernels, each owning its output rows.
//
//   dQ kernel  : CTA = 128 query rows; loops over the visible key tiles of 64
//       S  = Q K^T, dP = dO V^T            tcgen05.mma M128 N64 K64 each, fp32 in TMEM
//       dS = P o (dP - delta) / sqrt(hd)   thread = query row (TMEM lane), P = exp(S/sqrt(hd) - lse)
//       dQ += dS K                         A = dS (bf16, shared memory), B = K tile consumed MN-major
//   dK/dV kernel: CTA = 128 key rows; loops over the query tiles of 64 that can see them
//       S^T = K Q^T, dP^T = V dO^T         thread = key row
//       dV += P^T dO,  dK += dS^T Q        B = dO / Q tile consumed MN-major
// Operand tiles sit in shared memory in the canonical no-swizzle core-matrix layout (8 rows x 16
// bytes), staged with 16-byte cp.async (the upstream gradient arrives as bf16: the delta pre-pass
// converts an fp32 one once); one thread issues the MMAs, completion comes back through
// tcgen05.commit -> mbarrier, and every mbarrier wait is bounded exactly as in the forward
// kernel. A CTA has 256 threads: warps w and w+4 own the same 32 rows (TMEM lanes) and split the
// 64 columns of the score tiles between them. Two CTAs share an SM (256 TMEM columns each), so
// one CTA's exponentials overlap the other's MMAs.
#pragma once

#include "swa_tc.cuh"

namespace nlh {
namespace tc {

constexpr int BQ = 64;                       // query rows per step of the dK/dV kernel
constexpr int BTHREADS = 256;                // two warpgroups: columns [0,32) and [32,64) of a row
constexpr unsigned BWD_TMEM_COLS = 256;
constexpr float LOG2E = 1.4426950408889634f;

// dQ kernel shared memory
constexpr int DQ_OFF_Q = 0;
constexpr int DQ_OFF_DO = DQ_OFF_Q + Q_BYTES;
constexpr int DQ_OFF_K = DQ_OFF_DO + Q_BYTES;              // 2 buffers
constexpr int DQ_OFF_V = DQ_OFF_K + 2 * KV_BYTES;          // 2 buffers
constexpr int DQ_OFF_DS = DQ_OFF_V + 2 * KV_BYTES;
constexpr int DQ_OFF_BAR = DQ_OFF_DS + P_BYTES;
constexpr int DQ_OFF_TMEM = DQ_OFF_BAR + 16;
constexpr int DQ_SMEM_BYTES = DQ_OFF_TMEM + 16;

// dK/dV kernel shared memory
constexpr int KV_OFF_K = 0;                                // 128 rows
constexpr int KV_OFF_V = KV_OFF_K + Q_BYTES;
constexpr int KV_OFF_Q = KV_OFF_V + Q_BYTES;               // 2 buffers of 64 rows
constexpr int KV_OFF_DO = KV_OFF_Q + 2 * KV_BYTES;         // 2 buffers
constexpr int KV_OFF_P = KV_OFF_DO + 2 * KV_BYTES;
constexpr int KV_OFF_DS = KV_OFF_P + P_BYTES;
constexpr int KV_OFF_ROW = KV_OFF_DS + P_BYTES;            // [2][2][64] floats: lse*log2e | delta
constexpr int KV_OFF_BAR = KV_OFF_ROW + 2 * 2 * BQ * 4;
constexpr int KV_OFF_TMEM = KV_OFF_BAR + 16;
constexpr int KV_SMEM_BYTES = KV_OFF_TMEM + 16;

__device__ __forceinline__ bool visible(int qp, int kp, int window, int n_p)
{
    return kp <= qp && (kp < n_p || kp >= qp + 1 - window);
}

// stage_rows of the forward kernel for a CTA of BTHREADS threads.
__device__ __forceinline__ void stage_rows_b(unsigned char* dst, const __nv_bfloat16* __restrict__ src,
                                             size_t rs, int n_rows, int n_valid)
{
    for (int i = threadIdx.x; i < n_rows * 8; i += BTHREADS) {
        const int row = i >> 3, c = i & 7;
        unsigned char* d = dst + (row >> 3) * GROUP + c * CORE + (row & 7) * 16;
        if (row < n_valid) cp16_tc(d, src + (size_t)row * rs + c * 8);
        else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
}
__device__ __forceinline__ void cp4_tc(void* smem_dst, const void* gsrc)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
// 32 TMEM lanes x 32 consecutive 32-bit columns -> 32 registers.
__device__ __forceinline__ void tmem_ld_32x32b_x32(unsigned (&r)[32], unsigned taddr)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}

__device__ __forceinline__ void store_row8(float* dst, const float (&x)[8], bool accum)
{
    float4* p = reinterpret_cast<float4*>(dst);
    float4 a = make_float4(x[0], x[1], x[2], x[3]), b = make_float4(x[4], x[5], x[6], x[7]);
    if (accum) {
        const float4 o0 = p[0], o1 = p[1];
        a.x += o0.x; a.y += o0.y; a.z += o0.z; a.w += o0.w;
        b.x += o1.x; b.y += o1.y; b.z += o1.z; b.w += o1.w;
    }
    p[0] = a; p[1] = b;
}
__device__ __forceinline__ void store_row8(__nv_bfloat16* dst, const float (&x)[8], bool accum)
{
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; i++) y[i] = x[i] + (accum ? __bfloat162float(dst[i]) : 0.f);
    uint4 w;
    __nv_bfloat162 t0 = __floats2bfloat162_rn(y[0], y[1]), t1 = __floats2bfloat162_rn(y[2], y[3]);
    __nv_bfloat162 t2 = __floats2bfloat162_rn(y[4], y[5]), t3 = __floats2bfloat162_rn(y[6], y[7]);
    w.x = *reinterpret_cast<unsigned*>(&t0); w.y = *reinterpret_cast<unsigned*>(&t1);
    w.z = *reinterpret_cast<unsigned*>(&t2); w.w = *reinterpret_cast<unsigned*>(&t3);
    *reinterpret_cast<uint4*>(dst) = w;
}

// 8 fp32 values -> one 16-byte chunk of bf16
__device__ __forceinline__ uint4 pack8(const float (&p)[8])
{
    uint4 w;
    __nv_bfloat162 t0 = __floats2bfloat162_rn(p[0], p[1]), t1 = __floats2bfloat162_rn(p[2], p[3]);
    __nv_bfloat162 t2 = __floats2bfloat162_rn(p[4], p[5]), t3 = __floats2bfloat162_rn(p[6], p[7]);
    w.x = *reinterpret_cast<unsigned*>(&t0); w.y = *reinterpret_cast<unsigned*>(&t1);
    w.z = *reinterpret_cast<unsigned*>(&t2); w.w = *reinterpret_cast<unsigned*>(&t3);
    return w;
}

__device__ __forceinline__ void tmem_alloc_cols(unsigned char* slot, unsigned cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_free_cols(unsigned base, unsigned cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"(cols) : "memory");
}

// ───────────────────────────────── dQ ─────────────────────────────────────
// TMEM columns: S [0,64), dP [64,128), dQ [128,192). Thread (row = (warp & 3) * 32 + lane,
// half = warp >> 2) handles columns [32 half, 32 half + 32) of its row.
template <typename TG>
__global__ void __launch_bounds__(BTHREADS, 2) swa_bwd_dq_tc_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const __nv_bfloat16* __restrict__ d_out, const float* __restrict__ lse, const float* __restrict__ delta,
    TG* __restrict__ d_q, int S, int H, int window, int n_p, float scale, int rs_in, int rs_o)
{
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int half = warp >> 2, row = (warp & 3) * 32 + lane;
    const int qt = (gridDim.x - 1) - blockIdx.x;
    const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
    const size_t rs = (size_t)rs_in;
    const size_t base = (size_t)b * S * rs + (size_t)h * HD;
    const size_t base_o = (size_t)b * S * rs_o + (size_t)h * HD;
    const int q0 = qt * BM;
    const int q_hi = min(q0 + BM - 1, S - 1);
    const float sl2 = scale * LOG2E;
    const unsigned bar_s = smem_u32(smem + DQ_OFF_BAR), bar_o = bar_s + 8;
    volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(smem + DQ_OFF_TMEM);

    if (tid == 0) { mbar_init(bar_s, 1); mbar_init(bar_o, 1); }
    if (warp == 0) tmem_alloc_cols(smem + DQ_OFF_TMEM, BWD_TMEM_COLS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tmem_base = *tmem_slot;
    const unsigned tmem_row = tmem_base + ((unsigned)((warp & 3) * 32) << 16) + half * 32;

    const int kt_last = q_hi / BN;
    auto next_tile = [&](int cur) {
        for (int t = cur + 1; t <= kt_last; t++) {
            const int k_lo = t * BN;
            if (k_lo < n_p || k_lo + BN - 1 >= q0 + 1 - window) return t;
        }
        return -1;
    };
    auto load_kv = [&](int tile, int bufi) {
        const int k0 = tile * BN;
        stage_rows_b(smem + DQ_OFF_K + bufi * KV_BYTES, k + base + (size_t)k0 * rs, rs, BN, min(BN, S - k0));
        stage_rows_b(smem + DQ_OFF_V + bufi * KV_BYTES, v + base + (size_t)k0 * rs, rs, BN, min(BN, S - k0));
    };
    const unsigned idesc_kk = make_idesc(false), idesc_mn = make_idesc(true);
    const unsigned q_addr = smem_u32(smem + DQ_OFF_Q), do_addr = smem_u32(smem + DQ_OFF_DO);
    const unsigned ds_addr = smem_u32(smem + DQ_OFF_DS);
    auto issue_scores = [&](int bufi) {        // S = Q K^T -> cols [0,64); dP = dO V^T -> cols [64,128)
        const unsigned k_addr = smem_u32(smem + DQ_OFF_K + bufi * KV_BYTES);
        const unsigned v_addr = smem_u32(smem + DQ_OFF_V + bufi * KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++)
            mma_bf16(tmem_base, make_desc(q_addr + ks * 2 * CORE, CORE, GROUP),
                     make_desc(k_addr + ks * 2 * CORE, CORE, GROUP), idesc_kk, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++)
            mma_bf16(tmem_base + 64, make_desc(do_addr + ks * 2 * CORE, CORE, GROUP),
                     make_desc(v_addr + ks * 2 * CORE, CORE, GROUP), idesc_kk, ks > 0 ? 1u : 0u);
        mma_commit(bar_s);
    };

    int kt = next_tile(-1);
    stage_rows_b(smem + DQ_OFF_Q, q + base + (size_t)q0 * rs, rs, BM, min(BM, S - q0));
    stage_rows_b(smem + DQ_OFF_DO, d_out + base_o + (size_t)q0 * rs_o, (size_t)rs_o, BM, min(BM, S - q0));
    if (kt >= 0) load_kv(kt, 0);
    cp_commit_tc();
    const int qp = q0 + row;
    const size_t rowi = ((size_t)b * H + h) * S + min(qp, S - 1);
    const float lse2 = lse[rowi] * LOG2E;
    const float del = delta[rowi];
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    fence_async_proxy();
    fence_before_sync();
    __syncthreads();
    if (tid == 0 && kt >= 0) { fence_after_sync(); issue_scores(0); }

    unsigned par_s = 0, par_o = 0;
    bool dead = false;
    int it = 0;

    while (kt >= 0) {
        const int nxt = next_tile(kt);
        // A: this thread's 32 scores and 32 dP values of the tile
        if (!dead) dead = !mbar_wait(bar_s, par_s, WAIT_LIMIT);
        par_s ^= 1;
        fence_after_sync();
        unsigned sr[32], dr[32];
        tmem_ld_32x32b_x32(sr, tmem_row);
        tmem_ld_32x32b_x32(dr, tmem_row + 64);
        tmem_wait_ld();
        fence_before_sync();
        // B: the previous dQ update has consumed dS and its K tile
        if (it > 0) {
            if (!dead) dead = !mbar_wait(bar_o, par_o, WAIT_LIMIT);
            par_o ^= 1;
            fence_after_sync();
        }
        // C: prefetch the next K, V tiles (their buffers were last read by tile it-1)
        if (nxt >= 0) load_kv(nxt, (it + 1) & 1);
        cp_commit_tc();
        // E: dS = P o (dP - delta) * scale, written as bf16 in the K-major A layout
        const int k0 = kt * BN;
        const bool interior = (k0 + BN - 1 <= q0) && (k0 + BN - 1 < S) &&
                              ((k0 >= q0 + BM - window) || (k0 + BN - 1 < n_p));
        unsigned char* drow = smem + DQ_OFF_DS + (row >> 3) * GROUP + (row & 7) * 16 + half * 4 * CORE;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            float ds[8];
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const int j = c * 8 + e;
                float p = ex2_approx(fmaf(__uint_as_float(sr[j]), sl2, -lse2));
                if (!interior) {
                    const int kp = k0 + half * 32 + j;
                    if (!(qp < S && kp < S && visible(qp, kp, window, n_p))) p = 0.f;
                }
                ds[e] = p * (__uint_as_float(dr[j]) - del) * scale;
            }
            *reinterpret_cast<uint4*>(drow + c * CORE) = pack8(ds);
        }
        // F: dQ += dS K(it); then the next tile's scores
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        fence_async_proxy();
        fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            fence_after_sync();
            const unsigned k_addr = smem_u32(smem + DQ_OFF_K + (it & 1) * KV_BYTES);
#pragma unroll
            for (int ks = 0; ks < BN / 16; ks++)     // A = dS (K-major over keys), B = K tile (MN-major)
                mma_bf16(tmem_base + 128, make_desc(ds_addr + ks * 2 * CORE, CORE, GROUP),
                         make_desc(k_addr + ks * 2 * GROUP, GROUP, CORE), idesc_mn,
                         (it > 0 || ks > 0) ? 1u : 0u);
            mma_commit(bar_o);
            if (nxt >= 0) issue_scores((it + 1) & 1);
        }
        kt = nxt;
        it++;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    if (it > 0) {
        if (!dead) dead = !mbar_wait(bar_o, par_o, WAIT_LIMIT);
        fence_after_sync();
        unsigned orr[32];
        tmem_ld_32x32b_x32(orr, tmem_row + 128);
        tmem_wait_ld();
        if (qp < S) {
            TG* orow = d_q + base + (size_t)qp * rs + half * 32;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float x[8];
#pragma unroll
                for (int e = 0; e < 8; e++) x[e] = __uint_as_float(orr[c * 8 + e]);
                store_row8(orow + c * 8, x, false);
            }
        }
    } else if (qp < S) {
        TG* orow = d_q + base + (size_t)qp * rs + half * 32;
        const float z[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; c++) store_row8(orow + c * 8, z, false);
    }
    if (dead && lane == 0) atomicExch(&g_swa_tc_timeout, 1);
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_free_cols(tmem_base, BWD_TMEM_COLS);
}

// ─────────────────────────────── dK, dV ───────────────────────────────────
// TMEM columns: S^T [0,64), dP^T [64,128), dV [128,192), dK [192,256). Thread (row = key,
// half) handles query columns [32 half, 32 half + 32) of its key row.
template <typename TG, bool ACCUM>
__global__ void __launch_bounds__(BTHREADS, 2) swa_bwd_dkv_tc_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const __nv_bfloat16* __restrict__ d_out, const float* __restrict__ lse, const float* __restrict__ delta,
    TG* __restrict__ d_k, TG* __restrict__ d_v, int S, int H, int window, int n_p, float scale,
    int rs_in, int rs_o)
{
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int half = warp >> 2, row = (warp & 3) * 32 + lane;
    const int kt = blockIdx.x;
    const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
    const size_t rs = (size_t)rs_in;
    const size_t base = (size_t)b * S * rs + (size_t)h * HD;
    const size_t base_o = (size_t)b * S * rs_o + (size_t)h * HD;
    const int k0 = kt * BM;                                   // 128 keys per CTA
    const int k_hi = min(k0 + BM - 1, S - 1);
    const float sl2 = scale * LOG2E;
    const unsigned bar_s = smem_u32(smem + KV_OFF_BAR), bar_o = bar_s + 8;
    volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(smem + KV_OFF_TMEM);
    float* rowv = reinterpret_cast<float*>(smem + KV_OFF_ROW);        // [buf][lse | delta][64]

    if (tid == 0) { mbar_init(bar_s, 1); mbar_init(bar_o, 1); }
    if (warp == 0) tmem_alloc_cols(smem + KV_OFF_TMEM, BWD_TMEM_COLS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tmem_base = *tmem_slot;
    const unsigned tmem_row = tmem_base + ((unsigned)((warp & 3) * 32) << 16) + half * 32;

    // query tiles of 64: from the one holding k0 up to the last query that sees k_hi
    const int q_last = (k0 < n_p) ? (S - 1) : min(S - 1, k_hi + window - 1);
    const int qt_first = k0 / BQ, qt_last = q_last / BQ;
    const float* lse_bh = lse + ((size_t)b * H + h) * S;
    const float* del_bh = delta + ((size_t)b * H + h) * S;
    auto load_q = [&](int qtile, int bufi) {
        const int q0 = qtile * BQ, nq = min(BQ, S - q0);
        stage_rows_b(smem + KV_OFF_Q + bufi * KV_BYTES, q + base + (size_t)q0 * rs, rs, BQ, nq);
        stage_rows_b(smem + KV_OFF_DO + bufi * KV_BYTES, d_out + base_o + (size_t)q0 * rs_o, (size_t)rs_o, BQ, nq);
        if (tid < 2 * BQ) {                                   // lse and delta rows of the tile
            const int j = tid & (BQ - 1), which = tid >> 6;
            const int qp = min(q0 + j, S - 1);
            cp4_tc(rowv + (bufi * 2 + which) * BQ + j, (which ? del_bh : lse_bh) + qp);
        }
    };
    const unsigned idesc_kk = make_idesc(false), idesc_mn = make_idesc(true);
    const unsigned k_addr = smem_u32(smem + KV_OFF_K), v_addr = smem_u32(smem + KV_OFF_V);
    const unsigned p_addr = smem_u32(smem + KV_OFF_P), ds_addr = smem_u32(smem + KV_OFF_DS);
    auto issue_scores = [&](int bufi) {        // S^T = K Q^T -> [0,64); dP^T = V dO^T -> [64,128)
        const unsigned q_addr = smem_u32(smem + KV_OFF_Q + bufi * KV_BYTES);
        const unsigned do_addr = smem_u32(smem + KV_OFF_DO + bufi * KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++)
            mma_bf16(tmem_base, make_desc(k_addr + ks * 2 * CORE, CORE, GROUP),
                     make_desc(q_addr + ks * 2 * CORE, CORE, GROUP), idesc_kk, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++)
            mma_bf16(tmem_base + 64, make_desc(v_addr + ks * 2 * CORE, CORE, GROUP),
                     make_desc(do_addr + ks * 2 * CORE, CORE, GROUP), idesc_kk, ks > 0 ? 1u : 0u);
        mma_commit(bar_s);
    };

    stage_rows_b(smem + KV_OFF_K, k + base + (size_t)k0 * rs, rs, BM, min(BM, S - k0));
    stage_rows_b(smem + KV_OFF_V, v + base + (size_t)k0 * rs, rs, BM, min(BM, S - k0));
    load_q(qt_first, 0);
    cp_commit_tc();
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    fence_async_proxy();
    fence_before_sync();
    __syncthreads();
    if (tid == 0) { fence_after_sync(); issue_scores(0); }

    const int kp = k0 + row;
    unsigned par_s = 0, par_o = 0;
    bool dead = false;
    int it = 0;
    for (int qtile = qt_first; qtile <= qt_last; qtile++, it++) {
        const bool has_next = qtile < qt_last;
        const int bufi = it & 1;
        // A: this thread's part of S^T and dP^T
        if (!dead) dead = !mbar_wait(bar_s, par_s, WAIT_LIMIT);
        par_s ^= 1;
        fence_after_sync();
        unsigned sr[32], dr[32];
        tmem_ld_32x32b_x32(sr, tmem_row);
        tmem_ld_32x32b_x32(dr, tmem_row + 64);
        tmem_wait_ld();
        fence_before_sync();
        // B: the previous accumulation has consumed P, dS and its Q, dO tiles
        if (it > 0) {
            if (!dead) dead = !mbar_wait(bar_o, par_o, WAIT_LIMIT);
            par_o ^= 1;
            fence_after_sync();
        }
        // C: prefetch the next query tile into the buffer tile it-1 used
        if (has_next) load_q(qtile + 1, bufi ^ 1);
        cp_commit_tc();
        // E: P^T and dS^T of this key row for 32 queries
        const int q0 = qtile * BQ;
        const float* l2 = rowv + (bufi * 2 + 0) * BQ + half * 32;
        const float* dl = rowv + (bufi * 2 + 1) * BQ + half * 32;
        // every (query, key) pair of the tile visible: all queries at or after the last key, inside
        // the sequence, and the first key inside the window of the last query (or in the prefix)
        const bool interior = (q0 >= k0 + BM - 1) && (q0 + BQ - 1 < S) && (k0 + BM - 1 < S) &&
                              ((k0 >= q0 + BQ - window) || (k0 + BM - 1 < n_p));
        unsigned char* prow = smem + KV_OFF_P + (row >> 3) * GROUP + (row & 7) * 16 + half * 4 * CORE;
        unsigned char* drow = smem + KV_OFF_DS + (row >> 3) * GROUP + (row & 7) * 16 + half * 4 * CORE;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            float pp[8], ds[8];
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const int j = c * 8 + e;
                float p = ex2_approx(fmaf(__uint_as_float(sr[j]), sl2, -l2[j] * LOG2E));
                if (!interior) {
                    const int qp = q0 + half * 32 + j;
                    if (!(qp < S && kp < S && visible(qp, kp, window, n_p))) p = 0.f;
                }
                pp[e] = p;
                ds[e] = p * (__uint_as_float(dr[j]) - dl[j]) * scale;
            }
            *reinterpret_cast<uint4*>(prow + c * CORE) = pack8(pp);
            *reinterpret_cast<uint4*>(drow + c * CORE) = pack8(ds);
        }
        // F: dV += P^T dO, dK += dS^T Q; then the next tile's scores
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        fence_async_proxy();
        fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            fence_after_sync();
            const unsigned q_addr = smem_u32(smem + KV_OFF_Q + bufi * KV_BYTES);
            const unsigned do_addr = smem_u32(smem + KV_OFF_DO + bufi * KV_BYTES);
#pragma unroll
            for (int ks = 0; ks < BQ / 16; ks++)     // A = P^T (K-major over queries), B = dO tile (MN-major)
                mma_bf16(tmem_base + 128, make_desc(p_addr + ks * 2 * CORE, CORE, GROUP),
                         make_desc(do_addr + ks * 2 * GROUP, GROUP, CORE), idesc_mn, (it > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
            for (int ks = 0; ks < BQ / 16; ks++)     // A = dS^T, B = Q tile (MN-major)
                mma_bf16(tmem_base + 192, make_desc(ds_addr + ks * 2 * CORE, CORE, GROUP),
                         make_desc(q_addr + ks * 2 * GROUP, GROUP, CORE), idesc_mn, (it > 0 || ks > 0) ? 1u : 0u);
            mma_commit(bar_o);
            if (has_next) issue_scores(bufi ^ 1);
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    if (!dead) dead = !mbar_wait(bar_o, par_o, WAIT_LIMIT);
    fence_after_sync();
    {
        unsigned orr[32];
        tmem_ld_32x32b_x32(orr, tmem_row + 128);
        tmem_wait_ld();
        if (kp < S) {
            TG* orow = d_v + base + (size_t)kp * rs + half * 32;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float x[8];
#pragma unroll
                for (int e = 0; e < 8; e++) x[e] = __uint_as_float(orr[c * 8 + e]);
                store_row8(orow + c * 8, x, ACCUM);
            }
        }
        tmem_ld_32x32b_x32(orr, tmem_row + 192);
        tmem_wait_ld();
        if (kp < S) {
            TG* orow = d_k + base + (size_t)kp * rs + half * 32;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float x[8];
#pragma unroll
                for (int e = 0; e < 8; e++) x[e] = __uint_as_float(orr[c * 8 + e]);
                store_row8(orow + c * 8, x, ACCUM);
            }
        }
    }
    if (dead && lane == 0) atomicExch(&g_swa_tc_timeout, 1);
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_free_cols(tmem_base, BWD_TMEM_COLS);
}

}  // namespace tc
}  // namespace nlh
