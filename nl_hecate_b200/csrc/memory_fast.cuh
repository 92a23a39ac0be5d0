// Register-resident memory-rule kernels for head dimension D in {32, 64}.
//
// One CTA per independent (batch x head) problem. The D x D memory M (and the
// momentum S) never leave the register file during the sequence: D*D/16
// threads hold 16 elements each — one row, four float4 column chunks
// interleaved so that shared-memory reads of k/q are conflict-free and global
// state stores are full 32-byte sectors. Row reductions (M k, M q, dS k) are
// 1-3 warp shuffles inside the sequential dependency chain; column reductions
// (M^T dy, dS^T e), which only feed outputs, use a recursive-halving warp
// reduction and a deferred cross-warp sum per token tile. The k/v/q/dy/gate
// streams are staged tile by tile with 16-byte cp.async double buffering;
// backward state reads use a per-thread cp.async ring so no barrier sits in
// the token loop.
//
// Not covered here (generic kernels take over): error clip, Frobenius
// projection, other head dimensions, unaligned pointers, frozen chunks > 64.
#pragma once

#include "nlh_common.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {

constexpr int FAST_TT = 16;      // tokens per forward tile
constexpr int FAST_TB = 8;       // tokens per backward tile
constexpr int FAST_NST = 3;      // backward state ring depth (tokens)
constexpr int FAST_MAX_CHUNK = 64;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc)
{
    unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc)
{
    unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <int TPR>
__device__ __forceinline__ float row_allreduce(float v)
{
#pragma unroll
    for (int o = 1; o < TPR; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Column index (within a row of length D) of element i (0..15) held by column group cg.
template <int D>
__device__ __forceinline__ int col_of(int i, int cg) { return (i >> 2) * (D / 4) + cg * 4 + (i & 3); }

// Two-lane arithmetic on float2 values. Written as two scalar operations on purpose: the
// sm_100 packed-pair intrinsics (__ffma2_rn and friends) were measured on these kernels and
// lost — the compiler spent as many moves forming aligned register pairs as the packed
// instructions saved (same instruction total, 9 % longer run time).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y)); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return make_float2(a.x * b.x, a.y * b.y); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 bc2(float s) { return make_float2(s, s); }
__device__ __forceinline__ float2 shfl_xor2(float2 v, int o)
{
    return make_float2(__shfl_xor_sync(0xffffffffu, v.x, o), __shfl_xor_sync(0xffffffffu, v.y, o));
}

// A thread keeps its 16 elements of a row as 8 float2: pair p holds logical elements 2p, 2p+1;
// logical element i lives in 16-byte chunk i>>2. In the backward kernel the chunks are stored
// PERMUTED per lane: physical chunk j holds logical chunk j ^ xc, with
//   xc = 2*(lane bit 4) + (lane bit 3).
// With that layout the first two steps of the recursive-halving column reduction below always
// keep the low half of the registers and send the high half, so they need no selects.
__device__ __forceinline__ int chunk_perm(int lane) { return (((lane >> 4) & 1) << 1) | ((lane >> 3) & 1); }

// Recursive-halving reduction over the rows a warp owns. In: 16 per-thread column partials in
// the permuted layout. Out: NOUT = 16*TPR/32 fully warp-reduced values per lane, for the
// consecutive LOGICAL element indices base..base+NOUT-1 (same column chunk).
template <int TPR>
struct ColReduce {
    static constexpr int NOUT = 16 * TPR / 32;
    __device__ static __forceinline__ int base_index(int lane)
    {
        int b = 0;
        if (lane & 16) b += 8;
        if (TPR <= 8 && (lane & 8)) b += 4;
        if (TPR <= 4 && (lane & 4)) b += 2;
        if (TPR <= 2 && (lane & 2)) b += 1;
        return b;
    }
    __device__ static __forceinline__ void run(const float2 (&v)[8], int lane, float (&out)[NOUT])
    {
        static_assert(TPR == 4 || TPR == 2, "column reduction is written for 2 or 4 threads per row");
        float2 a4[4], a2[2];
#pragma unroll
        for (int i = 0; i < 4; i++) a4[i] = add2(v[i], shfl_xor2(v[i + 4], 16));   // lane bit 4 <-> chunk bit 1
#pragma unroll
        for (int i = 0; i < 2; i++) a2[i] = add2(a4[i], shfl_xor2(a4[i + 2], 8));  // lane bit 3 <-> chunk bit 0
        {   // lane bit 2 <-> pair within the chunk (not permuted: select)
            const bool up = lane & 4;
            const float2 send = up ? a2[0] : a2[1];
            const float2 keep = up ? a2[1] : a2[0];
            a2[0] = add2(keep, shfl_xor2(send, 4));
        }
        if (TPR == 4) {
            out[0] = a2[0].x;
            if (NOUT > 1) out[NOUT - 1] = a2[0].y;
            return;
        }
        {   // TPR == 2: lane bit 1 <-> element within the pair
            const bool up = lane & 2;
            const float send = up ? a2[0].x : a2[0].y;
            const float keep = up ? a2[0].y : a2[0].x;
            out[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
        }
    }
};

// SPLIT: CTAs per problem. The rows of M (and S) evolve independently of one another, so a problem's
// rows can be divided over SPLIT CTAs that share nothing but the k/v/q/gate streams they read;
// only the column sums (d_q, d_k) and the scalar gate gradients of the backward cross rows.
template <int D, int SPLIT = 1>
struct FastGeom {
    static constexpr int TPR = D / 16;          // threads per row
    static constexpr int ROWS = D / SPLIT;      // rows of the state owned by one CTA
    static constexpr int NT = ROWS * TPR;       // threads per CTA
    static constexpr int NW = NT / 32;          // warps
    static constexpr int RPW = 32 / TPR;        // rows per warp
};

// shared-memory floats
template <int D>
constexpr size_t fast_fwd_smem_floats() { return (size_t)3 * 2 * FAST_TT * D + 2 * 3 * FAST_TT + FAST_TT * D; }
// ring_mats: matrices per ring slot (2 when a stored S trajectory is read, else 1);
// frozen: the per-chunk error buffer is only needed by the frozen rules.
template <int D>
constexpr size_t fast_bwd_smem_floats(int ring_mats, bool frozen)
{
    using G = FastGeom<D>;
    return (size_t)4 * 2 * FAST_TB * D        // k,v,q,dy tiles, double buffered
         + 2 * 3 * FAST_TB                    // gates
         + (size_t)FAST_NST * ring_mats * D * D   // state ring
         + (size_t)2 * G::NW * FAST_TB * D    // dq / dk warp partials
         + (size_t)FAST_TB * D                // dv staging
         + (size_t)3 * FAST_TB * D            // per-row scalar partials
         + (frozen ? (size_t)FAST_MAX_CHUNK * D : 0);   // errors of the current chunk
}

// xc: chunk permutation of the calling thread (0 = logical order).
template <int D>
__device__ __forceinline__ void load_state8(float2 (&x)[8], const float* __restrict__ src, int r, int cg, int xc = 0)
{
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float4 t = *reinterpret_cast<const float4*>(src + (size_t)r * D + (j ^ xc) * (D / 4) + cg * 4);
        x[2 * j] = make_float2(t.x, t.y); x[2 * j + 1] = make_float2(t.z, t.w);
    }
}
template <int D>
__device__ __forceinline__ void store_state8(const float2 (&x)[8], float* dst, int r, int cg, int xc = 0)
{
#pragma unroll
    for (int j = 0; j < 4; j++)
        *reinterpret_cast<float4*>(dst + (size_t)r * D + (j ^ xc) * (D / 4) + cg * 4) =
            make_float4(x[2 * j].x, x[2 * j].y, x[2 * j + 1].x, x[2 * j + 1].y);
}
template <int D>
__device__ __forceinline__ void load_vec8(float2 (&x)[8], const float* src /*smem row of D*/, int cg, int xc = 0)
{
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float4 t = *reinterpret_cast<const float4*>(src + (j ^ xc) * (D / 4) + cg * 4);
        x[2 * j] = make_float2(t.x, t.y); x[2 * j + 1] = make_float2(t.z, t.w);
    }
}
__device__ __forceinline__ void zero8(float2 (&x)[8])
{
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = make_float2(0.f, 0.f);
}
__device__ __forceinline__ void copy8(float2 (&d)[8], const float2 (&s)[8])
{
#pragma unroll
    for (int i = 0; i < 8; i++) d[i] = s[i];
}
__device__ __forceinline__ float hsum8(const float2 (&x)[8])
{
    const float2 a = add2(add2(x[0], x[1]), add2(x[2], x[3]));
    const float2 b = add2(add2(x[4], x[5]), add2(x[6], x[7]));
    const float2 c = add2(a, b);
    return c.x + c.y;
}

// Cooperative async copy of ntok*D contiguous floats (16-byte pieces).
template <int D, int NT>
__device__ __forceinline__ void tile_async(float* dst, const float* __restrict__ src, int ntok)
{
    const int nvec = ntok * (D / 4);
    for (int i = threadIdx.x; i < nvec; i += NT) cp_async16(dst + 4 * i, src + 4 * i);
}

// ── bulk (TMA engine) staging of the stream tiles ──
// A tile of TT tokens of one stream is TT*D contiguous floats in global memory and in shared
// memory, so one thread can stage it with ONE bulk asynchronous copy whose completion is counted
// in bytes on an mbarrier (cp.async.bulk, the untiled form: both addresses 16-byte aligned, size a
// multiple of 16 bytes; plain single-CTA copies of this GPU's memory). Every thread then waits on
// the mbarrier phase instead of on its own cp.async group. Waits are bounded: when the limit runs
// out the CTA sets g_bulk_timeout and carries on (wrong results, no hang).
__device__ int g_bulk_timeout = 0;
constexpr unsigned BULK_WAIT_LIMIT = 1u << 22;
__device__ __forceinline__ unsigned smem_addr_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bulk_bar_init(unsigned bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void bulk_bar_expect(unsigned bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(unsigned dst, const void* src, unsigned bytes, unsigned bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool bulk_bar_wait(unsigned bar, unsigned parity)
{
    for (unsigned i = 0; i < BULK_WAIT_LIMIT; i++) {
        unsigned ok;
        asm volatile(
            "{\n\t"
            ".reg .pred P;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, P;\n\t"
            "}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// One forward token on register state. Msrc is the matrix the error is taken
// against (M itself, or the frozen chunk-start copy). Returns e (error or v for Hebbian).
template <int D, int RULE>
__device__ __forceinline__ float fast_fwd_token(float2 (&M)[8], float2 (&S)[8], const float2 (&Msrc)[8],
                                                const float* krow, float vr, float alpha, float theta,
                                                float eta, int cg, int xc = 0)
{
    constexpr int TPR = FastGeom<D>::TPR;
    float2 kk[8];
    load_vec8<D>(kk, krow, cg, xc);
    float e = vr;
    if (RULE != RULE_HEBBIAN) {
        float2 pa = make_float2(0.f, 0.f), pb = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            pa = fma2(Msrc[2 * i], kk[2 * i], pa);
            pb = fma2(Msrc[2 * i + 1], kk[2 * i + 1], pb);
        }
        const float2 ps = add2(pa, pb);
        e = row_allreduce<TPR>(ps.x + ps.y) - vr;
    }
    const float2 r2 = bc2(1.0f - alpha);
    if (RULE == RULE_TITANS) {
        const float2 nte = bc2(-theta * e), et2 = bc2(eta);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            S[i] = fma2(et2, S[i], mul2(nte, kk[i]));
            M[i] = fma2(r2, M[i], S[i]);
        }
    } else {
        const float2 c2 = bc2(RULE == RULE_DELTA ? -theta * e : e);
#pragma unroll
        for (int i = 0; i < 8; i++) M[i] = fma2(r2, M[i], mul2(c2, kk[i]));
    }
    return e;
}

template <int D>
__device__ __forceinline__ float fast_readout(const float2 (&M)[8], const float* qrow, int cg, int xc = 0)
{
    constexpr int TPR = FastGeom<D>::TPR;
    float2 qq[8];
    load_vec8<D>(qq, qrow, cg, xc);
    float2 ya = make_float2(0.f, 0.f), yb = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        ya = fma2(M[2 * i], qq[2 * i], ya);
        yb = fma2(M[2 * i + 1], qq[2 * i + 1], yb);
    }
    const float2 ys = add2(ya, yb);
    return row_allreduce<TPR>(ys.x + ys.y);
}

// D = 64, exact rules: capped at 64 registers so that four CTAs share an SM (the level-0 problem
// count of the stacked model, batch x heads = 512, then fits in one wave of 148 x 4).
// BULK: the k, v, q tiles are staged by thread 0 with bulk asynchronous copies (see above) instead
// of every thread's cp.async; the gates (4 bytes per token and stream) stay on cp.async.
template <int D, int RULE, bool FROZEN, int SPLIT = 1, bool BULK = false>
__global__ void __launch_bounds__(FastGeom<D, SPLIT>::NT, (D == 64 && !FROZEN) ? 4 : 1) fast_fwd_kernel(FwdArgs a)
{
    using G = FastGeom<D, SPLIT>;
    constexpr int NT = G::NT, TPR = G::TPR, TT = FAST_TT, ROWS = G::ROWS;
    extern __shared__ __align__(16) float sm[];
    __shared__ __align__(8) unsigned long long tile_bar[2];     // one mbarrier per tile buffer (BULK)
    float* kt = sm;
    float* vt = kt + 2 * TT * D;
    float* qt = vt + 2 * TT * D;
    float* gt = qt + 2 * TT * D;   // [2][3][TT]
    float* ys = gt + 2 * 3 * TT;   // [TT][ROWS]
    const int tid = threadIdx.x, cg = tid % TPR;
    const int part = (SPLIT > 1) ? (int)(blockIdx.x % SPLIT) : 0;
    const int r = part * ROWS + tid / TPR;       // global row of the state this thread holds
    const size_t dd = (size_t)D * D;
    const int b = blockIdx.x / SPLIT;
    const float* k = a.k + (size_t)b * a.in_stride_tok * D;
    const float* v = a.v + (size_t)b * a.in_stride_tok * D;
    const float* q = a.q + (size_t)b * a.in_stride_tok * D;
    const float* alpha = a.alpha + (size_t)b * a.in_stride_tok;
    const float* theta = (RULE != RULE_HEBBIAN) ? a.theta + (size_t)b * a.in_stride_tok : nullptr;
    const float* eta = (RULE == RULE_TITANS) ? a.eta + (size_t)b * a.in_stride_tok : nullptr;
    float* y = a.y + (size_t)b * a.seq_len * D;
    float* m_out = a.m_out + (size_t)b * a.out_stride;
    // s_out == NULL: the momentum trajectory is not stored (the backward derives S from M)
    float* s_out = (RULE == RULE_TITANS && a.s_out != nullptr) ? a.s_out + (size_t)b * a.out_stride : nullptr;
    const int mode = a.store_mode;

    float2 M[8], S[8], M0[8];
    load_state8<D>(M, a.m_init + (size_t)b * a.init_stride, r, cg);
    if (RULE == RULE_TITANS) load_state8<D>(S, a.s_init + (size_t)b * a.init_stride, r, cg);
    else zero8(S);
    copy8(M0, M);
    if (mode == STORE_ALL || mode == STORE_CKPT) {
        store_state8<D>(M, m_out, r, cg);
        if (RULE == RULE_TITANS && s_out != nullptr) store_state8<D>(S, s_out, r, cg);
    }

    const int ntiles = (a.seq_len + TT - 1) / TT;
    if (BULK) {
        if (tid == 0) { bulk_bar_init(smem_addr_u32(&tile_bar[0]), 1); bulk_bar_init(smem_addr_u32(&tile_bar[1]), 1); }
        __syncthreads();
    }
    bool bulk_dead = false;
    auto prefetch = [&](int tile) {
        const int t0 = tile * TT;
        const int ntok = min(TT, a.seq_len - t0);
        const int buf = tile & 1;
        if (BULK) {
            if (tid == 0) {
                const unsigned bar = smem_addr_u32(&tile_bar[buf]);
                const unsigned bytes = (unsigned)ntok * D * 4;
                bulk_bar_expect(bar, 3 * bytes);
                bulk_copy_g2s(smem_addr_u32(kt + buf * TT * D), k + (size_t)t0 * D, bytes, bar);
                bulk_copy_g2s(smem_addr_u32(vt + buf * TT * D), v + (size_t)t0 * D, bytes, bar);
                bulk_copy_g2s(smem_addr_u32(qt + buf * TT * D), q + (size_t)t0 * D, bytes, bar);
            }
        } else {
            tile_async<D, NT>(kt + buf * TT * D, k + (size_t)t0 * D, ntok);
            tile_async<D, NT>(vt + buf * TT * D, v + (size_t)t0 * D, ntok);
            tile_async<D, NT>(qt + buf * TT * D, q + (size_t)t0 * D, ntok);
        }
        if (tid < ntok) {
            cp_async4(gt + (buf * 3 + 0) * TT + tid, alpha + t0 + tid);
            if (RULE != RULE_HEBBIAN) cp_async4(gt + (buf * 3 + 1) * TT + tid, theta + t0 + tid);
            if (RULE == RULE_TITANS) cp_async4(gt + (buf * 3 + 2) * TT + tid, eta + t0 + tid);
        }
        cp_async_commit();
    };
    int slot = 1;
    if (ntiles > 0) prefetch(0);
    for (int tile = 0; tile < ntiles; tile++) {
        const int t0 = tile * TT;
        const int ntok = min(TT, a.seq_len - t0);
        const int buf = tile & 1;
        if (tile + 1 < ntiles) { prefetch(tile + 1); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        // BULK: buffer `buf` is used by tiles buf, buf + 2, ...: phase (tile >> 1) of its mbarrier
        if (BULK && !bulk_dead) bulk_dead = !bulk_bar_wait(smem_addr_u32(&tile_bar[buf]), (unsigned)(tile >> 1) & 1u);
        __syncthreads();
        const float* kb = kt + buf * TT * D;
        const float* vb = vt + buf * TT * D;
        const float* qb = qt + buf * TT * D;
        const float* gb = gt + buf * 3 * TT;
        for (int tl = 0; tl < ntok; tl++) {
            const int t = t0 + tl;
            if (mode == STORE_CHUNK && (t % a.interval) == 0) {
                const size_t off = (size_t)(t / a.interval) * dd;
                store_state8<D>(M, m_out + off, r, cg);
                if (RULE == RULE_TITANS && s_out != nullptr) store_state8<D>(S, s_out + off, r, cg);
                if (FROZEN) copy8(M0, M);
            } else if (FROZEN && mode == STORE_ALL && (t % a.interval) == 0) {
                copy8(M0, M);        // frozen rule with every state stored: interval = chunk size
            }
            const float al = gb[tl];
            const float th = (RULE != RULE_HEBBIAN) ? gb[TT + tl] : 0.f;
            const float et = (RULE == RULE_TITANS) ? gb[2 * TT + tl] : 0.f;
            if (FROZEN) fast_fwd_token<D, RULE>(M, S, M0, kb + tl * D, vb[tl * D + r], al, th, et, cg);
            else fast_fwd_token<D, RULE>(M, S, M, kb + tl * D, vb[tl * D + r], al, th, et, cg);
            if (mode == STORE_ALL) {
                store_state8<D>(M, m_out + (size_t)(t + 1) * dd, r, cg);
                if (RULE == RULE_TITANS && s_out != nullptr) store_state8<D>(S, s_out + (size_t)(t + 1) * dd, r, cg);
            } else if (mode == STORE_CKPT && (((t + 1) % a.interval) == 0 || t + 1 == a.seq_len)) {
                store_state8<D>(M, m_out + (size_t)slot * dd, r, cg);
                if (RULE == RULE_TITANS && s_out != nullptr) store_state8<D>(S, s_out + (size_t)slot * dd, r, cg);
                slot++;
            }
            const float yv = fast_readout<D>(M, qb + tl * D, cg);
            if (cg == 0) ys[tl * ROWS + (r - part * ROWS)] = yv;
        }
        __syncthreads();
        {
            // this CTA's ROWS entries of every output row
            const int nvec = ntok * (ROWS / 4);
            const float4* ysv = reinterpret_cast<const float4*>(ys);
            for (int i = tid; i < nvec; i += NT) {
                const int tl = i / (ROWS / 4), c = i - tl * (ROWS / 4);
                *reinterpret_cast<float4*>(y + (size_t)(t0 + tl) * D + part * ROWS + 4 * c) = ysv[i];
            }
        }
    }
    if (BULK && bulk_dead && tid == 0) atomicExch(&g_bulk_timeout, 1);
    if (mode == STORE_CHUNK) {
        const size_t off = (size_t)((a.seq_len + a.interval - 1) / a.interval) * dd;
        store_state8<D>(M, m_out + off, r, cg);
        if (RULE == RULE_TITANS && s_out != nullptr) store_state8<D>(S, s_out + off, r, cg);
    } else if (mode == STORE_FINAL) {
        store_state8<D>(M, m_out, r, cg);
        if (RULE == RULE_TITANS && s_out != nullptr) store_state8<D>(S, s_out, r, cg);
    }
}

// ───────────────────────────── backward ──────────────────────────────────
// Processes, in reverse, either the token range [t_start,t_end) against a
// stored trajectory (a.chunk == 0), or every chunk of a.chunk tokens with the
// chunk trajectory recomputed from its boundary state into scratch (m_rec).
// SDER (Titans, stored-trajectory mode only): no S trajectory is given; since
// S_{t+1} = M_{t+1} - (1-alpha_t) M_t and S_{t+1} = eta_t S_t - theta_t e k^T,
//   d_eta_t = <S_t, dS> = ( <M_{t+1} - (1-alpha_t) M_t, dS> + theta_t (e . dS k) ) / eta_t,
// which needs eta_t > 0 (gates far below ~1e-3 lose accuracy to the division).
template <int D, int RULE, bool FROZEN, bool SDER = false>
__global__ void __launch_bounds__(FastGeom<D>::NT, (D == 64 && !FROZEN) ? 2 : 1) fast_bwd_kernel(BwdArgs a)
{
    using G = FastGeom<D>;
    constexpr int NT = G::NT, TPR = G::TPR, NW = G::NW, TB = FAST_TB, NST = FAST_NST;
    constexpr int NOUT = ColReduce<TPR>::NOUT;
    extern __shared__ __align__(16) float sm[];
    float* kt = sm;                                   // [2][TB][D]
    float* vt = kt + 2 * TB * D;
    float* qt = vt + 2 * TB * D;
    float* dyt = qt + 2 * TB * D;
    float* gt = dyt + 2 * TB * D;                     // [2][3][TB]
    constexpr int RM = (RULE == RULE_TITANS && !SDER) ? 2 : 1;   // matrices per ring slot
    float* ring = gt + 2 * 3 * TB;                    // [NST][RM][D*D]
    float* pq = ring + (size_t)NST * RM * D * D;      // [NW][TB][D]
    float* pk = pq + (size_t)NW * TB * D;             // [NW][TB][D]
    float* dvs = pk + (size_t)NW * TB * D;            // [TB][D]
    float* scp = dvs + TB * D;                        // [3][TB][D] per-row partials
    float* es = scp + 3 * TB * D;                     // [FAST_MAX_CHUNK][D], frozen rules only

    const int tid = threadIdx.x, r = tid / TPR, cg = tid % TPR;
    const int lane = tid & 31, warp = tid >> 5;
    const size_t dd = (size_t)D * D;
    const int b = blockIdx.x;
    const size_t so = (size_t)b * a.seq_len * D, go = (size_t)b * a.seq_len;
    const float* k = a.k + so; const float* v = a.v + so; const float* q = a.q + so;
    const float* dy = a.d_y + so;
    float* dk = a.d_k + so; float* dv = a.d_v + so; float* dq = a.d_q + so;
    const float* alpha = a.alpha + go;
    const float* theta = (RULE != RULE_HEBBIAN) ? a.theta + go : nullptr;
    const float* eta = (RULE == RULE_TITANS) ? a.eta + go : nullptr;
    float* dalpha = a.d_alpha + go;
    float* dtheta = (RULE != RULE_HEBBIAN) ? a.d_theta + go : nullptr;
    float* deta = (RULE == RULE_TITANS) ? a.d_eta + go : nullptr;
    const float* mtraj = a.m_traj + (size_t)b * a.traj_stride;
    const float* straj = (RULE == RULE_TITANS && !SDER) ? a.s_traj + (size_t)b * a.traj_stride : nullptr;
    const bool recompute = a.chunk > 0;
    float* mrec = recompute ? a.m_rec + (size_t)b * (a.chunk + 1) * dd : nullptr;
    float* srec = (recompute && RULE == RULE_TITANS) ? a.s_rec + (size_t)b * (a.chunk + 1) * dd : nullptr;

    // All register state of this kernel uses the per-lane chunk permutation xc (see chunk_perm).
    const int xc = chunk_perm(lane);
    constexpr int DD = D * D;
    int co[4];   // float offsets, within a row, of the four chunks this thread holds
#pragma unroll
    for (int jj = 0; jj < 4; jj++) co[jj] = (jj ^ xc) * (D / 4) + cg * 4;
    float* const ring_t = ring + tid * 4;
    float2 dM[8], dS[8], dM0[8], M0[8], Mn[8];
    if (a.d_m_seed) load_state8<D>(dM, a.d_m_seed + (size_t)b * dd, r, cg, xc);
    else zero8(dM);
    if (RULE == RULE_TITANS && a.d_s_seed) load_state8<D>(dS, a.d_s_seed + (size_t)b * dd, r, cg, xc);
    else zero8(dS);
    zero8(dM0);
    zero8(M0);

    const int nchunks = recompute ? (a.seq_len + a.chunk - 1) / a.chunk : 1;
    for (int c = nchunks - 1; c >= 0; c--) {
        const int t0 = recompute ? c * a.chunk : a.t_start;
        const int t1 = recompute ? min(t0 + a.chunk, a.seq_len) : a.t_end;
        const int len = t1 - t0;
        const float* mt_base;   // slot j = state before token t0 + j
        const float* st_base;
        if (recompute) {
            // ── recompute the chunk trajectory into scratch (slots 0..len) ──
            float2 Mc[8], Sc[8];
            load_state8<D>(Mc, mtraj + (size_t)c * dd, r, cg, xc);
            if (RULE == RULE_TITANS) load_state8<D>(Sc, straj + (size_t)c * dd, r, cg, xc);
            else zero8(Sc);
            copy8(M0, Mc);
            store_state8<D>(Mc, mrec, r, cg, xc);
            if (RULE == RULE_TITANS) store_state8<D>(Sc, srec, r, cg, xc);
            const int ntl = (len + TB - 1) / TB;
            for (int tile = 0; tile < ntl; tile++) {
                const int tt0 = t0 + tile * TB;
                const int ntok = min(TB, t1 - tt0);
                __syncthreads();   // previous users of buffer 0 are done
                tile_async<D, NT>(kt, k + (size_t)tt0 * D, ntok);
                tile_async<D, NT>(vt, v + (size_t)tt0 * D, ntok);
                cp_async_commit();
                cp_async_wait<0>();
                __syncthreads();
                for (int tl = 0; tl < ntok; tl++) {
                    const int t = tt0 + tl;
                    const float al = alpha[t];
                    const float th = (RULE != RULE_HEBBIAN) ? theta[t] : 0.f;
                    const float et = (RULE == RULE_TITANS) ? eta[t] : 0.f;
                    float e;
                    if (FROZEN) e = fast_fwd_token<D, RULE>(Mc, Sc, M0, kt + tl * D, vt[tl * D + r], al, th, et, cg, xc);
                    else e = fast_fwd_token<D, RULE>(Mc, Sc, Mc, kt + tl * D, vt[tl * D + r], al, th, et, cg, xc);
                    if (FROZEN && cg == 0) es[(t - t0) * D + r] = e;
                    store_state8<D>(Mc, mrec + (size_t)(t - t0 + 1) * dd, r, cg, xc);
                    if (RULE == RULE_TITANS) store_state8<D>(Sc, srec + (size_t)(t - t0 + 1) * dd, r, cg, xc);
                }
            }
            __syncthreads();   // es visible; staging buffers free
            mt_base = mrec; st_base = srec;
            copy8(Mn, Mc);
            zero8(dM0);
        } else {
            mt_base = mtraj; st_base = straj;
            load_state8<D>(Mn, mt_base + (size_t)len * dd, r, cg, xc);
        }

        // ── reverse pass over the chunk, tile by tile ──
        const int ntl = (len + TB - 1) / TB;
        auto prefetch_tile = [&](int tile) {
            const int tt0 = t0 + tile * TB;
            const int ntok = min(TB, t1 - tt0);
            const int buf = tile & 1;
            tile_async<D, NT>(kt + buf * TB * D, k + (size_t)tt0 * D, ntok);
            tile_async<D, NT>(vt + buf * TB * D, v + (size_t)tt0 * D, ntok);
            tile_async<D, NT>(qt + buf * TB * D, q + (size_t)tt0 * D, ntok);
            tile_async<D, NT>(dyt + buf * TB * D, dy + (size_t)tt0 * D, ntok);
            if (tid < ntok) {
                cp_async4(gt + (buf * 3 + 0) * TB + tid, alpha + tt0 + tid);
                if (RULE != RULE_HEBBIAN) cp_async4(gt + (buf * 3 + 1) * TB + tid, theta + tt0 + tid);
                if (RULE == RULE_TITANS) cp_async4(gt + (buf * 3 + 2) * TB + tid, eta + tt0 + tid);
            }
        };
        // Thread-private async fetch of the next state slot, walking down from slot len-1 (slot
        // j = state before token t0+j). The ring is thread-major (piece jj of thread tid at
        // jj*NT*4 + tid*4): the data is private to the thread, so any layout works and this
        // one makes the 16-byte shared loads conflict-free. Ring slot = j mod NST, kept as a
        // counter; the global source pointer walks down by one state per call.
        int jp = len - 1;
        int pslot = (len > 0) ? (len - 1) % NST : 0;
        int cslot = pslot;
        const float* gpre = mt_base + (size_t)max(len - 1, 0) * DD + r * D;
        const ptrdiff_t sdiff = (RULE == RULE_TITANS && !SDER) ? (st_base - mt_base) : 0;
        auto prefetch_state = [&]() {
            if (jp >= 0) {
                float* dst = ring_t + pslot * (RM * DD);
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    cp_async16(dst + jj * NT * 4, gpre + co[jj]);
                    if (RULE == RULE_TITANS && !SDER) cp_async16(dst + DD + jj * NT * 4, gpre + sdiff + co[jj]);
                }
            }
            jp--;
            gpre -= DD;
            pslot = (pslot == 0) ? NST - 1 : pslot - 1;
        };
        if (len > 0) {
            // prologue: last tile + the first NST-1 states, one commit group each
            prefetch_tile(ntl - 1);
            prefetch_state();
            cp_async_commit();
#pragma unroll
            for (int s = 1; s < NST - 1; s++) { prefetch_state(); cp_async_commit(); }
        }
        for (int tile = ntl - 1; tile >= 0; tile--) {
            const int tt0 = t0 + tile * TB;
            const int ntok = min(TB, t1 - tt0);
            const int buf = tile & 1;
            const float* gb = gt + buf * 3 * TB;
            for (int tl = ntok - 1; tl >= 0; tl--) {
                const int j = tt0 + tl - t0;   // slot of M_t
                // keep NST-1 state groups in flight; fold the next tile's streams into this group
                prefetch_state();
                if (tl == ntok - 1 && tile > 0) prefetch_tile(tile - 1);
                cp_async_commit();
                // This tile's streams were committed at the first token of the tile processed
                // just before (tile+1). They are older than the NST-1 newest groups unless that
                // tile was shorter than the pipeline depth (only the sequence tail can be).
                if (tl == ntok - 1 && tile < ntl - 1 && (t1 - (tt0 + TB)) < NST) cp_async_wait<0>();
                else cp_async_wait<NST - 1>();
                if (tl == ntok - 1) __syncthreads();   // tile streams (other threads' copies) visible
                const float* ms = ring_t + cslot * (RM * DD);
                cslot = (cslot == 0) ? NST - 1 : cslot - 1;
                float2 Mt[8], St[8], kk[8], qq[8];
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    const float4 t4 = *reinterpret_cast<const float4*>(ms + jj * NT * 4);
                    Mt[2 * jj] = make_float2(t4.x, t4.y); Mt[2 * jj + 1] = make_float2(t4.z, t4.w);
                    if (RULE == RULE_TITANS && !SDER) {
                        const float4 s4 = *reinterpret_cast<const float4*>(ms + DD + jj * NT * 4);
                        St[2 * jj] = make_float2(s4.x, s4.y); St[2 * jj + 1] = make_float2(s4.z, s4.w);
                    }
                }
                // the k, v, q, dy tiles live in one array: row tl of buffer buf, constant strides
                const float* trow = kt + (buf * TB + tl) * D;
                constexpr int VOFF = 2 * TB * D, QOFF = 4 * TB * D, DYOFF = 6 * TB * D;
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    const float4 k4 = *reinterpret_cast<const float4*>(trow + co[jj]);
                    const float4 q4 = *reinterpret_cast<const float4*>(trow + QOFF + co[jj]);
                    kk[2 * jj] = make_float2(k4.x, k4.y); kk[2 * jj + 1] = make_float2(k4.z, k4.w);
                    qq[2 * jj] = make_float2(q4.x, q4.y); qq[2 * jj + 1] = make_float2(q4.z, q4.w);
                }
                const float dyr = trow[DYOFF + r];
                const float vr = trow[VOFF + r];
                const float al = gb[tl];
                const float th = (RULE != RULE_HEBBIAN) ? gb[TB + tl] : 0.f;
                const float et = (RULE == RULE_TITANS) ? gb[2 * TB + tl] : 0.f;
                const float rr = 1.0f - al;

                // pass 1: fold dy into dM (and dS); dot products of this row
                const float2 dy2 = bc2(dyr), nrr2 = bc2(-rr);
                float2 p2 = make_float2(0.f, 0.f), ua = make_float2(0.f, 0.f), ub = make_float2(0.f, 0.f);
                float2 pa2 = make_float2(0.f, 0.f), pe2 = make_float2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    dM[i] = fma2(dy2, qq[i], dM[i]);
                    float2 g = dM[i];
                    if (RULE == RULE_TITANS) {
                        dS[i] = add2(dS[i], dM[i]);
                        g = dS[i];
                        if (SDER) pe2 = fma2(fma2(nrr2, Mt[i], Mn[i]), dS[i], pe2);   // S_{t+1} = M_{t+1} - (1-alpha) M_t
                        else pe2 = fma2(St[i], dS[i], pe2);
                    }
                    pa2 = fma2(Mt[i], dM[i], pa2);
                    if (RULE != RULE_HEBBIAN && !FROZEN) p2 = fma2(Mt[i], kk[i], p2);
                    if (i & 1) ub = fma2(g, kk[i], ub); else ua = fma2(g, kk[i], ua);
                }
                const float2 us = add2(ua, ub);
                const float u = row_allreduce<TPR>(us.x + us.y);
                float e = 0.f;
                if (RULE != RULE_HEBBIAN) {
                    if (FROZEN) e = es[j * D + r];
                    else e = row_allreduce<TPR>(p2.x + p2.y) - vr;
                }
                const float de = -th * u;
                // per-row scalar partials (summed over the rows at tile end)
                const float pa = row_allreduce<TPR>(pa2.x + pa2.y);
                float pe = 0.f;
                if (RULE == RULE_TITANS) pe = row_allreduce<TPR>(pe2.x + pe2.y);
                if (cg == 0) {
                    scp[(0 * TB + tl) * D + r] = pa;
                    scp[(1 * TB + tl) * D + r] = (RULE != RULE_HEBBIAN) ? e * u : 0.f;
                    if (SDER) pe = (et > 1e-30f) ? __fdividef(pe + th * e * u, et) : 0.f;
                    scp[(2 * TB + tl) * D + r] = pe;
                    dvs[tl * D + r] = (RULE == RULE_HEBBIAN) ? u : th * u;
                }

                // pass 2: column partials d_q = M_{t+1}^T dy ; d_k = -theta G^T e + Mk^T de
                // (Hebbian: dM^T v), then propagate dM / dS to the previous token
                float2 cq[8], ck[8];
                const float2 de2 = bc2(de), nthe2 = bc2(-th * e), vr2 = bc2(vr), et2 = bc2(et), rr2 = bc2(rr);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    cq[i] = mul2(Mn[i], dy2);
                    if (RULE == RULE_HEBBIAN) ck[i] = mul2(dM[i], vr2);
                    else ck[i] = fma2((RULE == RULE_TITANS) ? dS[i] : dM[i], nthe2, mul2(FROZEN ? M0[i] : Mt[i], de2));
                    if (RULE == RULE_TITANS) dS[i] = mul2(dS[i], et2);
                    float2 dm = mul2(dM[i], rr2);
                    if (RULE != RULE_HEBBIAN) {
                        if (FROZEN) dM0[i] = fma2(kk[i], de2, dM0[i]);
                        else dm = fma2(kk[i], de2, dm);
                    }
                    dM[i] = dm;
                    Mn[i] = Mt[i];
                }
                float oq[NOUT], ok[NOUT];
                ColReduce<TPR>::run(cq, lane, oq);
                ColReduce<TPR>::run(ck, lane, ok);
                {
                    const int bi = ColReduce<TPR>::base_index(lane);
                    const int pcol = (warp * TB + tl) * D + col_of<D>(bi, cg);
#pragma unroll
                    for (int i = 0; i < NOUT; i++) { pq[pcol + i] = oq[i]; pk[pcol + i] = ok[i]; }
                }
            }
            __syncthreads();
            // ── tile epilogue: cross-warp sums and coalesced stores ──
            for (int i = tid; i < ntok * D; i += NT) {
                float sq = 0.f, sk = 0.f;
#pragma unroll
                for (int w = 0; w < NW; w++) { sq += pq[(size_t)w * TB * D + i]; sk += pk[(size_t)w * TB * D + i]; }
                dq[(size_t)tt0 * D + i] = sq;
                dk[(size_t)tt0 * D + i] = sk;
                dv[(size_t)tt0 * D + i] = dvs[i];
            }
            for (int job = warp; job < 3 * ntok; job += NW) {
                const int which = job / ntok, tl = job - which * ntok;
                if ((which == 1 && RULE == RULE_HEBBIAN) || (which == 2 && RULE != RULE_TITANS)) continue;
                float s = 0.f;
                for (int i = lane; i < D; i += 32) s += scp[(which * TB + tl) * D + i];
                s = warp_sum(s);
                if (lane == 0) {
                    if (which == 0) dalpha[tt0 + tl] = -s;
                    else if (which == 1) dtheta[tt0 + tl] = -s;
                    else deta[tt0 + tl] = s;
                }
            }
            // the next tile's first-token barrier orders these reads before pq/pk/scp are rewritten
        }
        if (FROZEN) {
#pragma unroll
            for (int i = 0; i < 8; i++) dM[i] = add2(dM[i], dM0[i]);
        }
        __syncthreads();
    }

    if (a.atomic_out) {
        if (a.d_m_out == nullptr) return;   // batch-summed initial-state gradients not requested
#pragma unroll
        for (int i = 0; i < 8; i++) {
            // physical pair i holds logical elements 2i ^ (xc << 2) and the next one
            const size_t o = (size_t)r * D + col_of<D>((2 * i) ^ (xc << 2), cg);
            atomicAdd(&a.d_m_out[o], dM[i].x);
            atomicAdd(&a.d_m_out[o + 1], dM[i].y);
            if (RULE == RULE_TITANS) { atomicAdd(&a.d_s_out[o], dS[i].x); atomicAdd(&a.d_s_out[o + 1], dS[i].y); }
        }
    } else {
        store_state8<D>(dM, a.d_m_out + (size_t)b * dd, r, cg, xc);
        if (RULE == RULE_TITANS) store_state8<D>(dS, a.d_s_out + (size_t)b * dd, r, cg, xc);
    }
}

// ───────────────────────────── host dispatch ─────────────────────────────
inline bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

inline bool fast_common_ok(int d, float clip, float mmax)
{
    return (d == 64 || d == 32) && !(clip > 0.0f) && !m_norm_enabled(mmax);
}

// Number of SMs of the current device (queried once per process).
inline int sm_count()
{
    static int n = 0;
    if (n == 0) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) n = v;
        else n = 148;
    }
    return n;
}
// With at most half as many problems as SMs, every problem's rows are divided over two CTAs, each
// on an SM of its own: the run time of these kernels is then set by the per-token dependency
// chain of one CTA, not by throughput, and half the rows per CTA shortens it (measured at 64
// problems of 512 tokens: forward 0.27 -> 0.19 ms, M-only backward 0.48 -> 0.42 ms; with 128
// problems two CTAs would share an SM and nothing is gained).
inline bool split_rows(int d, int batch) { return d == 64 && 2 * batch <= sm_count() && option_value(NLH_OPT_ROW_SPLIT) != 0; }

template <int D, int RULE>
static bool fast_fwd_launch(const FwdArgs& a, cudaStream_t st)
{
    const size_t smem = fast_fwd_smem_floats<D>() * sizeof(float);
    if constexpr (D == 64) {
        if (!a.frozen && split_rows(a.d, a.batch)) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(fast_fwd_kernel<D, RULE, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            fast_fwd_kernel<D, RULE, false, 2><<<a.batch * 2, FastGeom<D, 2>::NT, smem, st>>>(a);
            return true;
        }
    }
    // bulk staging of the stream tiles: every tile starts on a 16-byte boundary (bases checked by
    // the caller; token rows are D * 4 = 128 or 256 bytes)
    if (option_value(NLH_OPT_BULK_STAGING)) {
        if (a.frozen) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(fast_fwd_kernel<D, RULE, true, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            fast_fwd_kernel<D, RULE, true, 1, true><<<a.batch, FastGeom<D>::NT, smem, st>>>(a);
        } else {
            if (smem > 48 * 1024) cudaFuncSetAttribute(fast_fwd_kernel<D, RULE, false, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            fast_fwd_kernel<D, RULE, false, 1, true><<<a.batch, FastGeom<D>::NT, smem, st>>>(a);
        }
        return true;
    }
    if (a.frozen) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(fast_fwd_kernel<D, RULE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fast_fwd_kernel<D, RULE, true><<<a.batch, FastGeom<D>::NT, smem, st>>>(a);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(fast_fwd_kernel<D, RULE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fast_fwd_kernel<D, RULE, false><<<a.batch, FastGeom<D>::NT, smem, st>>>(a);
    }
    return true;
}

// Returns true when a fast kernel was launched (caller checks the launch).
static bool fast_forward(int rule, const FwdArgs& a, cudaStream_t st)
{
    if (!fast_common_ok(a.d, a.error_clip, a.m_norm_max)) return false;
    if (a.frozen && rule == RULE_HEBBIAN) return false;
    const bool al = aligned16(a.k) && aligned16(a.v) && aligned16(a.q) && aligned16(a.y) &&
                    aligned16(a.m_init) && aligned16(a.m_out) &&
                    (rule != RULE_TITANS || (aligned16(a.s_init) && aligned16(a.s_out))) &&
                    (a.s_out != nullptr || rule != RULE_TITANS || a.store_mode == STORE_ALL) &&
                    (a.init_stride % 4 == 0) && (a.out_stride % 4 == 0);
    if (!al) return false;
    if (a.d == 64) {
        if (rule == RULE_TITANS) return fast_fwd_launch<64, RULE_TITANS>(a, st);
        if (rule == RULE_DELTA) return fast_fwd_launch<64, RULE_DELTA>(a, st);
        if (rule == RULE_HEBBIAN) return fast_fwd_launch<64, RULE_HEBBIAN>(a, st);
    } else {
        if (rule == RULE_TITANS) return fast_fwd_launch<32, RULE_TITANS>(a, st);
        if (rule == RULE_DELTA) return fast_fwd_launch<32, RULE_DELTA>(a, st);
        if (rule == RULE_HEBBIAN) return fast_fwd_launch<32, RULE_HEBBIAN>(a, st);
    }
    return false;
}

// Exact Titans backward on an M-only trajectory (defined in memory_exact_bwd.cuh).
template <int D>
static bool exact_bwd_launch(const BwdArgs& a, cudaStream_t st);

template <int D, int RULE>
static bool fast_bwd_launch(const BwdArgs& a, cudaStream_t st)
{
    const bool sder = (RULE == RULE_TITANS && a.s_traj == nullptr);
    const size_t smem = fast_bwd_smem_floats<D>((RULE == RULE_TITANS && !sder) ? 2 : 1, a.frozen) * sizeof(float);
    if (sder) return exact_bwd_launch<D>(a, st);   // checked by the caller: stored-trajectory mode
    if (a.frozen) {
        cudaFuncSetAttribute(fast_bwd_kernel<D, RULE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fast_bwd_kernel<D, RULE, true><<<a.batch, FastGeom<D>::NT, smem, st>>>(a);
    } else {
        cudaFuncSetAttribute(fast_bwd_kernel<D, RULE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fast_bwd_kernel<D, RULE, false><<<a.batch, FastGeom<D>::NT, smem, st>>>(a);
    }
    return true;
}

static bool fast_backward(int rule, BwdArgs& a, cudaStream_t st)
{
    if (!fast_common_ok(a.d, a.error_clip, a.m_norm_max)) return false;
    if (a.frozen && (rule == RULE_HEBBIAN || a.chunk > FAST_MAX_CHUNK)) return false;
    if (a.t_end <= a.t_start && a.chunk <= 0) return false;
    const bool al = aligned16(a.k) && aligned16(a.v) && aligned16(a.q) && aligned16(a.d_y) &&
                    aligned16(a.d_k) && aligned16(a.d_v) && aligned16(a.d_q) && aligned16(a.m_traj) &&
                    (rule != RULE_TITANS || aligned16(a.s_traj)) && (a.traj_stride % 4 == 0) &&
                    (a.s_traj != nullptr || rule != RULE_TITANS || (a.chunk <= 0 && !a.frozen)) &&
                    aligned16(a.d_m_out) && (rule != RULE_TITANS || aligned16(a.d_s_out)) &&
                    (a.d_m_seed == nullptr || aligned16(a.d_m_seed)) &&
                    (a.d_s_seed == nullptr || aligned16(a.d_s_seed));
    if (!al) return false;
    if (a.chunk > 0) {
        const size_t dd = (size_t)a.d * a.d;
        const size_t per = (((size_t)a.batch * (a.chunk + 1) * dd * sizeof(float)) + 255) & ~(size_t)255;
        char* ws = (char*)workspace(per * 2);
        if (!ws) return false;
        a.m_rec = (float*)ws;
        a.s_rec = (float*)(ws + per);
    }
    if (a.d == 64) {
        if (rule == RULE_TITANS) return fast_bwd_launch<64, RULE_TITANS>(a, st);
        if (rule == RULE_DELTA) return fast_bwd_launch<64, RULE_DELTA>(a, st);
        if (rule == RULE_HEBBIAN) return fast_bwd_launch<64, RULE_HEBBIAN>(a, st);
    } else {
        if (rule == RULE_TITANS) return fast_bwd_launch<32, RULE_TITANS>(a, st);
        if (rule == RULE_DELTA) return fast_bwd_launch<32, RULE_DELTA>(a, st);
        if (rule == RULE_HEBBIAN) return fast_bwd_launch<32, RULE_HEBBIAN>(a, st);
    }
    return false;
}

}  // namespace nlh
