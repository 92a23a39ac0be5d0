// SWA forward on the 5th-generation tensor cores (tcgen05) with TMEM accumulators, head_dim 64.
//
// One CTA = 128 query rows of one (batch, head); key tiles of 64. Per key tile:
//   S  = Q K^T   : tcgen05.mma kind::f16, M=128 N=64 K=64 (4 instructions), fp32 in TMEM cols [0,64)
//   softmax      : every thread owns ONE query row (TMEM lane = row): tcgen05.ld 32x32b.x64 gives
//                  the thread its 64 scores, so max / exp / sum need no shuffles at all
//   P (bf16)     : written to shared memory in the tensor core's K-major core-matrix layout
//   PV = P V     : tcgen05.mma M=128 N=64 K=64, V consumed MN-major straight from its tile,
//                  accumulated across key tiles in TMEM cols [64,128); when a row's running
//                  maximum moves, its warp rescales the accumulator in place (tcgen05.ld / st)
// Operands are staged into canonical no-swizzle core-matrix layouts (8 rows x 16 bytes contiguous)
// either by tiled TMA copies issued by one thread (TMA variant: one cp.async.bulk.tensor per
// 8-element chunk column of a tile, completion counted on an mbarrier) or by 16-byte cp.async of
// every thread; K and V tiles are double buffered and the score MMA of tile i+1 is issued before
// the softmax of tile i so the two overlap.
// A single thread issues the MMAs; completion is tracked with tcgen05.commit -> mbarrier. Every
// mbarrier wait is bounded: on expiry the CTA sets a global error flag, stops waiting, frees its
// TMEM and returns.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace nlh {
namespace tc {

constexpr int BM = 128;          // query rows per CTA
constexpr int BN = 64;           // keys per tile
constexpr int HD = 64;
constexpr int THREADS = 128;
constexpr unsigned TMEM_COLS = 128;
constexpr unsigned WAIT_LIMIT = 1u << 20;

// shared-memory byte offsets
constexpr int Q_BYTES = BM * HD * 2;        // 16 KB
constexpr int KV_BYTES = BN * HD * 2;       // 8 KB
constexpr int P_BYTES = BM * BN * 2;        // 16 KB
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + Q_BYTES;              // 2 buffers
constexpr int OFF_V = OFF_K + 2 * KV_BYTES;         // 2 buffers
constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
constexpr int OFF_BAR = OFF_P + P_BYTES;            // four 8-byte mbarriers (S ready, O updated, two tile-load stages)
constexpr int OFF_TMEM = OFF_BAR + 32;              // 4-byte TMEM base address
constexpr int SMEM_BYTES = OFF_TMEM + 16;

// Canonical no-swizzle core-matrix layouts (core matrix = 8 rows x 16 bytes, contiguous):
//  K-major operand (rows = M or N index, 16-byte chunks along K):
//     byte(row, kchunk) = (row/8) * SBO + kchunk * LBO + (row%8) * 16,  LBO = 128, SBO = 8*128
//  MN-major operand (V: "rows" of a core matrix are 8 consecutive K indices = keys, the 16 bytes
//  are 8 consecutive N indices = head-dim elements):
//     byte(key, nchunk) = (key/8) * LBO + nchunk * SBO + (key%8) * 16,  SBO = 128, LBO = 8*128
constexpr unsigned CORE = 128;
constexpr unsigned GROUP = (HD / 8) * CORE;   // 1024: one 8-row (or 8-key) group of 8 core matrices

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// 64-bit shared-memory matrix descriptor, SWIZZLE_NONE, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_desc(unsigned smem_addr, unsigned lbo_bytes, unsigned sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
// Instruction descriptor: D fp32, A/B bf16, M=128, N=64; b_mn_major selects the B layout.
__device__ __forceinline__ unsigned make_idesc(bool b_mn_major)
{
    unsigned d = 0;
    d |= 1u << 4;                 // D format F32
    d |= 1u << 7;                 // A format BF16
    d |= 1u << 10;                // B format BF16
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= (unsigned)(BN >> 3) << 17;
    d |= (unsigned)(BM >> 4) << 24;
    return d;
}

__device__ __forceinline__ void mma_bf16(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc,
                                         unsigned accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned bar_addr)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(bar_addr) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ void mbar_init(unsigned bar_addr, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar_addr), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
// Bounded wait on a phase parity. Returns false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned bar_addr, unsigned parity, unsigned limit)
{
    for (unsigned i = 0; i < limit; i++) {
        unsigned ok;
        asm volatile(
            "{\n\t"
            ".reg .pred P;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, P;\n\t"
            "}\n"
            : "=r"(ok) : "r"(bar_addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// 32 TMEM lanes (one per thread of the warp) x 64 consecutive 32-bit columns -> 64 registers.
__device__ __forceinline__ void tmem_ld_32x32b_x64(unsigned (&r)[64], unsigned taddr)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
                 : "r"(taddr));
}

// 64 registers -> 32 TMEM lanes x 64 consecutive columns (inverse of tmem_ld_32x32b_x64).
__device__ __forceinline__ void tmem_st_32x32b_x64(unsigned taddr, const unsigned (&r)[64])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x64.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63, %64};\n"
                 :
                 : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(r[32]), "r"(r[33]), "r"(r[34]), "r"(r[35]), "r"(r[36]), "r"(r[37]), "r"(r[38]), "r"(r[39]), "r"(r[40]), "r"(r[41]), "r"(r[42]), "r"(r[43]), "r"(r[44]), "r"(r[45]), "r"(r[46]), "r"(r[47]), "r"(r[48]), "r"(r[49]), "r"(r[50]), "r"(r[51]), "r"(r[52]), "r"(r[53]), "r"(r[54]), "r"(r[55]), "r"(r[56]), "r"(r[57]), "r"(r[58]), "r"(r[59]), "r"(r[60]), "r"(r[61]), "r"(r[62]), "r"(r[63])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void cp16_tc(void* smem_dst, const void* gsrc)
{
    unsigned s = smem_u32(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_commit_tc() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }

// ── TMA staging (TMA = true variant of the forward kernel) ──
// The operand tiles are then laid out chunk-major: 16-byte chunk c of row r at c * (rows * 16) +
// r * 16, i.e. one contiguous column of `rows` x 16 bytes per chunk of 8 head-dim elements. That is
// still a canonical no-swizzle core-matrix layout (8 rows x 16 bytes contiguous), only with the
// two descriptor strides exchanged (K-chunk stride rows * 16, 8-row-group stride 128), and it is
// what a tiled TMA copy with a box of {8 elements, rows} writes: one cp.async.bulk.tensor per
// chunk, issued by one thread, completion counted in bytes on an mbarrier. The tensor maps are
// 3-D {head-dim elements of all heads, sequence positions, batch}: rows past the end of the
// sequence are out of bounds of the map and arrive as zeros. Every copy is a plain single-CTA load.
__device__ __forceinline__ void mbar_expect_tx(unsigned bar_addr, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar_addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_3d(unsigned smem_dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            unsigned bar_addr)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar_addr)
        : "memory");
}
// One tile of `rows` rows x 64 head-dim elements of head h, starting at sequence position row0 of
// batch element b: 8 copies of {8 elements, rows}. c0 = h*64 + 8*c is a multiple of 8 bf16 = 16 bytes.
__device__ __forceinline__ void tma_tile(unsigned smem_dst, const CUtensorMap* map, int h, int row0, int b,
                                         int rows, unsigned bar_addr)
{
#pragma unroll
    for (int c = 0; c < HD / 8; c++)
        tma_load_3d(smem_dst + c * rows * 16, map, h * HD + 8 * c, row0, b, bar_addr);
}

// Stage n_rows rows of 64 bf16 (row stride rs elements) into the core-matrix layout:
// 16-byte chunk c of row r goes to (r/8)*GROUP + c*CORE + (r%8)*16. Rows >= n_valid are zeroed.
__device__ __forceinline__ void stage_rows(unsigned char* dst, const __nv_bfloat16* __restrict__ src,
                                           size_t rs, int n_rows, int n_valid)
{
    for (int i = threadIdx.x; i < n_rows * 8; i += THREADS) {
        const int row = i >> 3, c = i & 7;
        unsigned char* d = dst + (row >> 3) * GROUP + c * CORE + (row & 7) * 16;
        if (row < n_valid) cp16_tc(d, src + (size_t)row * rs + c * 8);
        else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
}

__device__ int g_swa_tc_timeout = 0;   // set when a bounded mbarrier wait ran out

// Pipeline per key tile i (S and O live in TMEM, columns [0,64) and [64,128)):
//   A  wait S(i) ready, every thread pulls its row of 64 scores into registers
//   B  wait PV(i-1) done  -> P buffer, V(i-1) buffer and O are free
//   C  prefetch K(i+2) and V(i+1) with cp.async (K two tiles ahead, V one tile ahead: two
//      buffers each are enough because K(i) is dead once S(i) is ready)
//   D  barrier; one thread issues S(i+1) = Q K(i+1)^T  -> runs under the softmax of tile i
//   E  softmax of tile i in registers (masks only on boundary tiles), P -> shared memory;
//      O is rescaled in TMEM only by warps whose running maximum moved (tcgen05.ld/st)
//   F  barrier; one thread issues O += P V(i)
// TMA = true: Q, K and V tiles are staged by thread 0 with tiled TMA copies (see above) instead of
// every thread's cp.async; only that thread waits for them (it is the one that issues the MMAs
// that read them), on two alternating mbarriers with bounded waits.
template <bool TMA>
__global__ void __launch_bounds__(THREADS) swa_fwd_tc_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
    const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
    int S, int H, int window, int n_p, float scale, int rs_in, int rs_o,
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v)
{
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5;
    const int qt = (gridDim.x - 1) - blockIdx.x;
    const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
    const size_t rs = (size_t)rs_in;                       // row stride of q, k, v (elements)
    const size_t base = (size_t)b * S * rs + (size_t)h * HD;
    const size_t base_o = (size_t)b * S * rs_o + (size_t)h * HD;   // output rows
    const int q0 = qt * BM;
    const int q_hi = min(q0 + BM - 1, S - 1);
    const float sl2 = scale * 1.4426950408889634f;
    const unsigned bar_s = smem_u32(smem + OFF_BAR), bar_o = bar_s + 8, bar_ld = bar_s + 16;   // bar_ld, bar_ld + 8
    volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(smem + OFF_TMEM);

    if (tid == 0) {
        mbar_init(bar_s, 1); mbar_init(bar_o, 1);
        if (TMA) { mbar_init(bar_ld, 1); mbar_init(bar_ld + 8, 1); }
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(smem + OFF_TMEM)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tmem_base = *tmem_slot;
    const unsigned tmem_row = tmem_base + ((unsigned)(warp * 32) << 16);   // this warp's 32 lanes

    const int kt_last = q_hi / BN;
    auto next_tile = [&](int cur) {
        for (int t = cur + 1; t <= kt_last; t++) {
            const int k_lo = t * BN;
            if (k_lo < n_p || k_lo + BN - 1 >= q0 + 1 - window) return t;
        }
        return -1;
    };
    // cp.async variant: every thread stages its part; TMA variant: thread 0 issues the copies onto
    // the mbarrier ld_bar given by the caller
    auto load_k = [&](int tile, int bufi, unsigned ld_bar) {
        const int k0 = tile * BN;
        if (TMA) { if (tid == 0) tma_tile(smem_u32(smem + OFF_K + bufi * KV_BYTES), &map_k, h, k0, b, BN, ld_bar); }
        else stage_rows(smem + OFF_K + bufi * KV_BYTES, k + base + (size_t)k0 * rs, rs, BN, min(BN, S - k0));
    };
    auto load_v = [&](int tile, int bufi, unsigned ld_bar) {
        const int k0 = tile * BN;
        if (TMA) { if (tid == 0) tma_tile(smem_u32(smem + OFF_V + bufi * KV_BYTES), &map_v, h, k0, b, BN, ld_bar); }
        else stage_rows(smem + OFF_V + bufi * KV_BYTES, v + base + (size_t)k0 * rs, rs, BN, min(BN, S - k0));
    };
    const unsigned idesc_qk = make_idesc(false), idesc_pv = make_idesc(true);
    const unsigned q_addr = smem_u32(smem + OFF_Q), p_addr = smem_u32(smem + OFF_P);
    // descriptor strides of the staged operands: (stride between K chunks, stride between 8-row groups)
    constexpr unsigned Q_LBO = TMA ? BM * 16 : CORE, Q_SBO = TMA ? CORE : GROUP;
    constexpr unsigned K_LBO = TMA ? BN * 16 : CORE, K_SBO = TMA ? CORE : GROUP;
    // V is consumed MN-major: (stride between 8-key groups, stride between head-dim chunks)
    constexpr unsigned V_KG = TMA ? CORE : GROUP, V_NC = TMA ? BN * 16 : CORE;
    auto issue_qk = [&](int bufi) {     // S = Q K^T, both operands K-major, 2 chunks per K=16 step
        const unsigned k_addr = smem_u32(smem + OFF_K + bufi * KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++)
            mma_bf16(tmem_base, make_desc(q_addr + ks * 2 * Q_LBO, Q_LBO, Q_SBO),
                     make_desc(k_addr + ks * 2 * K_LBO, K_LBO, K_SBO), idesc_qk, ks > 0 ? 1u : 0u);
        mma_commit(bar_s);
    };

    int kt = next_tile(-1);
    int nxt = (kt >= 0) ? next_tile(kt) : -1;
    bool dead = false;
    if (TMA) {
        // load group 0 on bar_ld: Q, K(0), V(0), K(1); group it+1 (issued in iteration it) goes to
        // bar_ld + 8 * ((it + 1) & 1) and is waited for by thread 0 in iteration it+1
        if (tid == 0) {
            const unsigned bytes = Q_BYTES + (kt >= 0 ? 2 * KV_BYTES : 0) + (nxt >= 0 ? KV_BYTES : 0);
            mbar_expect_tx(bar_ld, bytes);
            tma_tile(q_addr, &map_q, h, q0, b, BM, bar_ld);
        }
        if (kt >= 0) { load_k(kt, 0, bar_ld); load_v(kt, 0, bar_ld); }
        if (nxt >= 0) load_k(nxt, 1, bar_ld);
        if (tid == 0) {
            dead = !mbar_wait(bar_ld, 0, WAIT_LIMIT);
            if (kt >= 0) { fence_after_sync(); issue_qk(0); }
        }
    } else {
        stage_rows(smem + OFF_Q, q + base + (size_t)q0 * rs, rs, BM, min(BM, S - q0));
        if (kt >= 0) { load_k(kt, 0, 0); load_v(kt, 0, 0); }
        if (nxt >= 0) load_k(nxt, 1, 0);
        cp_commit_tc();
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        fence_async_proxy();
        fence_before_sync();
        __syncthreads();
        if (tid == 0 && kt >= 0) { fence_after_sync(); issue_qk(0); }
    }

    float m_run = -INFINITY, l_run = 0.f;
    const int qp = q0 + tid;
    unsigned par_s = 0, par_o = 0;
    int it = 0;

    while (kt >= 0) {
        const int nxt2 = (nxt >= 0) ? next_tile(nxt) : -1;
        // A: scores of this tile
        if (!dead) dead = !mbar_wait(bar_s, par_s, WAIT_LIMIT);
        par_s ^= 1;
        fence_after_sync();
        unsigned sr[64];
        tmem_ld_32x32b_x64(sr, tmem_row);
        tmem_wait_ld();
        fence_before_sync();
        // B: previous P V product has been folded into O
        if (it > 0) {
            if (!dead) dead = !mbar_wait(bar_o, par_o, WAIT_LIMIT);
            par_o ^= 1;
            fence_after_sync();
        }
        // C: prefetch
        if (TMA) {
            const unsigned ld_next = bar_ld + 8 * ((it + 1) & 1);
            if (tid == 0 && nxt >= 0) mbar_expect_tx(ld_next, (nxt2 >= 0 ? KV_BYTES : 0) + KV_BYTES);
            if (nxt2 >= 0) load_k(nxt2, it & 1, ld_next);       // K(it+2) over K(it)
            if (nxt >= 0) load_v(nxt, (it + 1) & 1, ld_next);   // V(it+1) over V(it-1)
            // D: thread 0 waits for load group `it` (K(it+1), V(it)); the barrier is for the S
            // columns, which every thread has read by now
            if (tid == 0 && it > 0 && !dead) dead = !mbar_wait(bar_ld + 8 * (it & 1), (unsigned)(it >> 1) & 1u, WAIT_LIMIT);
        } else {
            if (nxt2 >= 0) load_k(nxt2, it & 1, 0);            // K(it+2) over K(it)
            if (nxt >= 0) load_v(nxt, (it + 1) & 1, 0);        // V(it+1) over V(it-1)
            cp_commit_tc();
            // D: K(it+1) (committed one tile ago) has landed; start the next score tile
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
            fence_async_proxy();
        }
        fence_before_sync();
        __syncthreads();
        if (tid == 0 && nxt >= 0) { fence_after_sync(); issue_qk((it + 1) & 1); }

        // E: softmax
        const int k0 = kt * BN;
        const bool interior = (k0 + BN - 1 <= q0) && (k0 + BN - 1 < S) &&
                              ((k0 >= q0 + BM - window) || (k0 + BN - 1 < n_p));
        float mx = -INFINITY;
        if (interior) {
#pragma unroll
            for (int j = 0; j < BN; j++) mx = fmaxf(mx, __uint_as_float(sr[j]));
        } else {
#pragma unroll
            for (int j = 0; j < BN; j++) {
                const int kp = k0 + j;
                const bool ok = kp < S && kp <= qp && (kp < n_p || kp >= qp + 1 - window);
                const float s = ok ? __uint_as_float(sr[j]) : -INFINITY;
                sr[j] = __float_as_uint(s);
                mx = fmaxf(mx, s);
            }
        }
        const float m_new = fmaxf(m_run, mx);
        const float mu = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = ex2_approx((m_run - mu) * sl2);
        const bool moved = (m_new != m_run);
        m_run = m_new;
        const float mus = mu * sl2;
        float ls = 0.f;
        unsigned char* prow = smem + OFF_P + (tid >> 3) * GROUP + (tid & 7) * 16;
#pragma unroll
        for (int c = 0; c < BN / 8; c++) {
            float p[8];
#pragma unroll
            for (int e = 0; e < 8; e++) {
                p[e] = ex2_approx(fmaf(__uint_as_float(sr[c * 8 + e]), sl2, -mus));
                ls += p[e];
            }
            uint4 w;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(p[0], p[1]), t1 = __floats2bfloat162_rn(p[2], p[3]);
            __nv_bfloat162 t2 = __floats2bfloat162_rn(p[4], p[5]), t3 = __floats2bfloat162_rn(p[6], p[7]);
            w.x = *reinterpret_cast<unsigned*>(&t0); w.y = *reinterpret_cast<unsigned*>(&t1);
            w.z = *reinterpret_cast<unsigned*>(&t2); w.w = *reinterpret_cast<unsigned*>(&t3);
            *reinterpret_cast<uint4*>(prow + c * CORE) = w;
        }
        l_run = l_run * corr + ls;
        // rescale O in TMEM, only in warps where some row's maximum moved (never on the first tile:
        // O is not initialised yet and the first product overwrites it)
        if (it > 0 && __any_sync(0xffffffffu, moved)) {
            tmem_ld_32x32b_x64(sr, tmem_row + 64);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < HD; j++) sr[j] = __float_as_uint(__uint_as_float(sr[j]) * corr);
            tmem_st_32x32b_x64(tmem_row + 64, sr);
            tmem_wait_st();
        }
        // F: O (+)= P V
        fence_async_proxy();
        fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            fence_after_sync();
            const unsigned v_addr = smem_u32(smem + OFF_V + (it & 1) * KV_BYTES);
#pragma unroll
            for (int ks = 0; ks < BN / 16; ks++)      // A = P (K-major over keys), B = V (MN-major)
                mma_bf16(tmem_base + 64, make_desc(p_addr + ks * 2 * CORE, CORE, GROUP),
                         make_desc(v_addr + ks * 2 * V_KG, V_KG, V_NC), idesc_pv,
                         (it > 0 || ks > 0) ? 1u : 0u);
            mma_commit(bar_o);
        }
        kt = nxt;
        nxt = nxt2;
        it++;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    if (it > 0) {
        if (!dead) dead = !mbar_wait(bar_o, par_o, WAIT_LIMIT);
        fence_after_sync();
        unsigned orr[64];
        tmem_ld_32x32b_x64(orr, tmem_row + 64);
        tmem_wait_ld();
        if (qp < S) {
            const float inv = (l_run > 0.f) ? 1.0f / l_run : 0.f;
            __nv_bfloat16* orow = out + base_o + (size_t)qp * rs_o;
#pragma unroll
            for (int c = 0; c < HD / 8; c++) {
                uint4 w;
                __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(orr[c * 8]) * inv, __uint_as_float(orr[c * 8 + 1]) * inv);
                __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(orr[c * 8 + 2]) * inv, __uint_as_float(orr[c * 8 + 3]) * inv);
                __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(orr[c * 8 + 4]) * inv, __uint_as_float(orr[c * 8 + 5]) * inv);
                __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(orr[c * 8 + 6]) * inv, __uint_as_float(orr[c * 8 + 7]) * inv);
                w.x = *reinterpret_cast<unsigned*>(&t0); w.y = *reinterpret_cast<unsigned*>(&t1);
                w.z = *reinterpret_cast<unsigned*>(&t2); w.w = *reinterpret_cast<unsigned*>(&t3);
                *reinterpret_cast<uint4*>(orow + c * 8) = w;
            }
            if (lse != nullptr) lse[((size_t)b * H + h) * S + qp] = m_run * scale + logf(l_run);
        }
    }
    if (dead && (tid & 31) == 0) atomicExch(&g_swa_tc_timeout, 1);
    fence_before_sync();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
}

}  // namespace tc
}  // namespace nlh
