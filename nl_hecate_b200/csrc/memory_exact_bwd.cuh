// Exact (per-token) Titans backward against a stored M trajectory only — the level-0 kernel of
// the stacked model. Same mathematics as fast_bwd_kernel<D, RULE_TITANS, false, true>
// (S_{t+1} is rebuilt as M_{t+1} - (1-alpha_t) M_t), restructured so that no state matrix is
// carried between tokens:
//
//   iteration t            first half : load M_t; row dots <M_t,dM>, <M_t,dS>, M_t k, dS k;
//                                       d_k column partials; dS *= eta; dM = (1-alpha) dM + de k^T
//                          second half: (for token t-1, while M_t is still in registers)
//                                       dM += dy q^T; dS += dM; <M_t,dS>; d_q column partials = M_t^T dy
//
// i.e. everything token t-1 needs from M_t = "its M_{t+1}" is taken in iteration t, so M_{t+1} is
// never copied forward (16 registers and 16 moves per token less than the generic kernel) and
// 2 CTAs of 128 registers fit per SM without spills. The second half of a tile's top token runs
// before the tile's loop, after the previous tile's epilogue, so every partial row of a tile is
// produced between two of its own barriers.
#pragma once

#include "memory_fast.cuh"

namespace nlh {

template <int D, int SPLIT = 1, bool FROZEN = false>
constexpr size_t exact_bwd_smem_floats()
{
    using G = FastGeom<D, SPLIT>;
    return (FROZEN ? (size_t)G::ROWS * D : 0)  // chunk-start state (frozen rule)
         + (size_t)2 * FAST_TB * 4 * D        // k | v | q | dy rows, double buffered
         + 2 * FAST_TB * 4                    // gates (alpha, theta, eta, pad)
         + (size_t)FAST_NST * G::ROWS * D     // state ring (M only, this CTA's rows)
         + (size_t)2 * G::NW * FAST_TB * D    // dq / dk warp partials
         + (size_t)FAST_TB * G::ROWS          // dv staging
         + (size_t)3 * FAST_TB * G::ROWS;     // per-row scalar partials
}

// SPLIT = 2: the problem's rows are divided over two CTAs (see FastGeom). Each CTA then holds
// partial column sums and partial gate gradients, which it ADDS into d_q, d_k, d_alpha, d_theta,
// d_eta with atomicAdd (two addends per element: the result does not depend on their order); the
// launcher zeroes those five outputs first.
// FROZEN: the frozen-M0 chunkwise rule on a FULL stored M trajectory (every token's state, as the
// exact rule stores it) instead of a recomputed chunk window: inside a chunk of a.chunk tokens the
// error reads the chunk-start state M_c (e_t = M_c k_t - v_t), so d_k takes M_c^T de, the de k^T
// terms collect in dM0 and join dM when the walk reaches the chunk's first token
// (core/kernels/titans_chunkwise_backward.cu:196-351). Everything else — the S derivation from
// consecutive M states included — is the exact rule's. M_c (16 registers) and dM0 (16) leave room
// for one CTA per SM; the chunk-start state of the NEXT chunk is fetched with cp.async into a
// thread-private buffer while the current chunk is processed.
template <int D, int SPLIT = 1, bool FROZEN = false>
__global__ void __launch_bounds__(FastGeom<D, SPLIT>::NT, FROZEN ? 1 : (D == 64 ? (SPLIT == 1 ? 2 : 3) : 8)) titans_exact_bwd_kernel(BwdArgs a)
{
    static_assert(!FROZEN || SPLIT == 1, "the frozen variant is not row-split");
    using G = FastGeom<D, SPLIT>;
    constexpr int NT = G::NT, TPR = G::TPR, NW = G::NW, TB = FAST_TB, NST = FAST_NST, DD = D * D;
    constexpr int ROWS = G::ROWS, RD = ROWS * D;      // floats of one state slot held by this CTA
    constexpr int NOUT = ColReduce<TPR>::NOUT;
    constexpr int ROW = 4 * D;                        // staged floats per token: k | v | q | dy
    constexpr int VOFF = D, QOFF = 2 * D, DYOFF = 3 * D;
    extern __shared__ __align__(16) float sm[];
    float* tiles = sm;                                // [2][TB][ROW]
    float* gt = tiles + 2 * TB * ROW;                 // [2][TB][4]
    float* ring = gt + 2 * TB * 4;                    // [NST][RD], thread-major pieces
    float* pq = ring + (size_t)NST * RD;              // [NW][TB][D]
    float* pk = pq + (size_t)NW * TB * D;             // [NW][TB][D]
    float* dvs = pk + (size_t)NW * TB * D;            // [TB][ROWS]
    float* scp = dvs + TB * ROWS;                     // [3][TB][ROWS]
    float* mcb = scp + 3 * TB * ROWS;                 // [RD] chunk-start state, thread-major (FROZEN)

    const int tid = threadIdx.x, rl = tid / TPR, cg = tid % TPR;   // rl: row within this CTA
    const int part = (SPLIT > 1) ? (int)(blockIdx.x % SPLIT) : 0;
    const int r = part * ROWS + rl;                                // global row of the state
    const int lane = tid & 31, warp = tid >> 5;
    const int xc = chunk_perm(lane);
    int co[4];   // float offsets, within a row, of the four chunks this thread holds
#pragma unroll
    for (int jj = 0; jj < 4; jj++) co[jj] = (jj ^ xc) * (D / 4) + cg * 4;
    float* const ring_t = ring + tid * 4;
    const int bi = ColReduce<TPR>::base_index(lane);
    const int wcol = warp * TB * D + col_of<D>(bi, cg);   // this lane's slot in a partial row

    const int b = blockIdx.x / SPLIT;
    const size_t so = (size_t)b * a.seq_len * D, go = (size_t)b * a.seq_len;
    const float* k = a.k + so; const float* v = a.v + so; const float* q = a.q + so;
    const float* dy = a.d_y + so;
    const int t0 = a.t_start, t1 = a.t_end, len = t1 - t0;
    const float* mt_base = a.m_traj + (size_t)b * a.traj_stride;   // slot j = state before token t0+j

    float2 dM[8], dS[8], Mt[8];
    float2 Mc[8], dM0[8];                             // FROZEN only: chunk-start state, its gradient terms
    float* const mcb_t = mcb + tid * 4;
    const int C = FROZEN ? a.chunk : 1;
    int cs_next = -1;                                 // chunk start whose state is to be fetched next
    int cs_age = NST;                                 // commit groups since the last fetch was issued
    auto prefetch_chunk_state = [&](int cs) {         // state before token cs (trajectory slot cs)
        const float* src = mt_base + (size_t)(cs - t0) * DD + r * D;
#pragma unroll
        for (int jj = 0; jj < 4; jj++) cp_async16(mcb_t + jj * NT * 4, src + co[jj]);
        cs_age = 0;
    };
    auto load_chunk_state = [&]() {
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const float4 t4 = *reinterpret_cast<const float4*>(mcb_t + jj * NT * 4);
            Mc[2 * jj] = make_float2(t4.x, t4.y); Mc[2 * jj + 1] = make_float2(t4.z, t4.w);
        }
    };
    if (FROZEN) zero8(dM0);
    if (a.d_m_seed) load_state8<D>(dM, a.d_m_seed + (size_t)b * DD, r, cg, xc);
    else zero8(dM);
    if (a.d_s_seed) load_state8<D>(dS, a.d_s_seed + (size_t)b * DD, r, cg, xc);
    else zero8(dS);

    const int ntl = (len + TB - 1) / TB;
    auto prefetch_tile = [&](int tile) {
        const int tt0 = t0 + tile * TB;
        const int ntok = min(TB, t1 - tt0);
        float* tb = tiles + (tile & 1) * TB * ROW;
        const int np = ntok * (D / 4);                 // 16-byte pieces per stream
        for (int i = tid; i < np; i += NT) {
            const int tl = i / (D / 4), c = i - tl * (D / 4);
            const size_t src = (size_t)(tt0 + tl) * D + c * 4;
            float* dst = tb + tl * ROW + c * 4;
            cp_async16(dst, k + src);
            cp_async16(dst + VOFF, v + src);
            cp_async16(dst + QOFF, q + src);
            cp_async16(dst + DYOFF, dy + src);
        }
        if (tid < ntok) {
            float* g = gt + ((tile & 1) * TB + tid) * 4;
            cp_async4(g, a.alpha + go + tt0 + tid);
            cp_async4(g + 1, a.theta + go + tt0 + tid);
            cp_async4(g + 2, a.eta + go + tt0 + tid);
        }
    };
    // state ring: slots len, len-1, ..., 0 in this order; slot index mod NST kept as a counter
    int jp = len;
    int pslot = len % NST;
    int cslot = pslot;
    const float* gpre = mt_base + (size_t)max(len, 0) * DD + r * D;
    auto prefetch_state = [&]() {
        if (jp >= 0) {
            float* dst = ring_t + pslot * RD;
#pragma unroll
            for (int jj = 0; jj < 4; jj++) cp_async16(dst + jj * NT * 4, gpre + co[jj]);
        }
        jp--;
        gpre -= DD;
        pslot = (pslot == 0) ? NST - 1 : pslot - 1;
    };
    auto load_state = [&]() {     // consume the oldest state in flight into Mt
        const float* ms = ring_t + cslot * RD;
        cslot = (cslot == 0) ? NST - 1 : cslot - 1;
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const float4 t4 = *reinterpret_cast<const float4*>(ms + jj * NT * 4);
            Mt[2 * jj] = make_float2(t4.x, t4.y); Mt[2 * jj + 1] = make_float2(t4.z, t4.w);
        }
    };

    float2 pea = make_float2(0.f, 0.f);   // per-thread part of <M_{t+1}, dS> for the coming token
    // Second half for the token staged at `row`, tile-local index tl; Mt holds its M_{t+1}.
    auto second_half = [&](const float* row, int tl) {
        float2 qq[8], cq[8];
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const float4 q4 = *reinterpret_cast<const float4*>(row + QOFF + co[jj]);
            qq[2 * jj] = make_float2(q4.x, q4.y); qq[2 * jj + 1] = make_float2(q4.z, q4.w);
        }
        const float2 dy2 = bc2(row[DYOFF + r]);
        pea = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            dM[i] = fma2(dy2, qq[i], dM[i]);
            dS[i] = add2(dS[i], dM[i]);
            pea = fma2(Mt[i], dS[i], pea);
            cq[i] = mul2(Mt[i], dy2);
        }
        float oq[NOUT];
        ColReduce<TPR>::run(cq, lane, oq);
#pragma unroll
        for (int i = 0; i < NOUT; i++) pq[wcol + tl * D + i] = oq[i];
    };

    if (len > 0) {
        prefetch_tile(ntl - 1);
        if (FROZEN) prefetch_chunk_state(((t1 - 1) / C) * C);   // the last chunk's start, first group
        prefetch_state();            // state len, same group as the last tile
        cp_async_commit();
        prefetch_state();            // state len-1
        cp_async_commit();
        prefetch_state();            // state len-2
        cp_async_commit();
        cp_async_wait<NST - 1>();    // first group landed
        __syncthreads();             // ... for every thread: the tile is visible
        cs_age = NST;                // ... and so has the last chunk's start state
        load_state();                // Mt = M_len
    }
    for (int tile = ntl - 1; tile >= 0; tile--) {
        const int tt0 = t0 + tile * TB;
        const int ntok = min(TB, t1 - tt0);
        const float* tb = tiles + (tile & 1) * TB * ROW;
        const float* gb = gt + (tile & 1) * TB * 4;
        // top token of the tile: its M_{t+1} is the state loaded last
        second_half(tb + (ntok - 1) * ROW, ntok - 1);
        for (int tl = ntok - 1; tl >= 0; tl--) {
            // keep NST-1 state groups in flight; the next tile's streams ride in the first group
            prefetch_state();
            if (tl == ntok - 1 && tile > 0) prefetch_tile(tile - 1);
            if (FROZEN && cs_next >= 0) { prefetch_chunk_state(cs_next); cs_next = -1; }
            cp_async_commit();
            cp_async_wait<NST - 1>();
            load_state();            // Mt = M_t
            if (FROZEN) {
                const int t = tt0 + tl;
                cs_age++;
                if (t == t1 - 1 || (t + 1) % C == 0) {       // first token processed of its chunk
                    if (cs_age < NST) cp_async_wait<0>();    // a short chunk: the fetch may still be in flight
                    load_chunk_state();
                    const int cs = (t / C) * C;
                    cs_next = (cs - C >= t0) ? cs - C : -1;  // fetched from the next iteration on
                }
            }
            const float* row = tb + tl * ROW;
            float2 kk[8];
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                const float4 k4 = *reinterpret_cast<const float4*>(row + co[jj]);
                kk[2 * jj] = make_float2(k4.x, k4.y); kk[2 * jj + 1] = make_float2(k4.z, k4.w);
            }
            const float vr = row[VOFF + r];
            const float4 gate = *reinterpret_cast<const float4*>(gb + tl * 4);
            const float al = gate.x, th = gate.y, et = gate.z;
            const float rr = 1.0f - al;

            float2 ua = make_float2(0.f, 0.f), ub = make_float2(0.f, 0.f), p2 = make_float2(0.f, 0.f);
            float2 pa2 = make_float2(0.f, 0.f), pb2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (i & 1) ub = fma2(dS[i], kk[i], ub); else ua = fma2(dS[i], kk[i], ua);
                p2 = fma2(FROZEN ? Mc[i] : Mt[i], kk[i], p2);
                pa2 = fma2(Mt[i], dM[i], pa2);
                pb2 = fma2(Mt[i], dS[i], pb2);
            }
            const float2 us = add2(ua, ub);
            const float u = row_allreduce<TPR>(us.x + us.y);          // (dS k)_r
            const float de = -th * u;
            const float e = row_allreduce<TPR>(p2.x + p2.y) - vr;     // (M_t k - v)_r
            const float pa = row_allreduce<TPR>(pa2.x + pa2.y);       // <M_t, dM>_r
            // <S_{t+1}, dS>_r = <M_{t+1}, dS>_r - (1-alpha) <M_t, dS>_r
            const float ps = row_allreduce<TPR>((pea.x + pea.y) - rr * (pb2.x + pb2.y));
            if (cg == 0) {
                scp[(0 * TB + tl) * ROWS + rl] = pa;
                scp[(1 * TB + tl) * ROWS + rl] = e * u;
                // d_eta_t = <S_t, dS> with S_t = (S_{t+1} + theta e k^T) / eta
                scp[(2 * TB + tl) * ROWS + rl] = (et > 1e-30f) ? __fdividef(ps + th * e * u, et) : 0.f;
                dvs[tl * ROWS + rl] = th * u;
            }
            {
                float2 ck[8];
                const float2 de2 = bc2(de), nthe2 = bc2(-th * e), et2 = bc2(et), rr2 = bc2(rr);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    ck[i] = fma2(dS[i], nthe2, mul2(FROZEN ? Mc[i] : Mt[i], de2));   // d_k = -theta dS^T e + M^T de
                    dS[i] = mul2(dS[i], et2);
                    if (FROZEN) { dM0[i] = fma2(kk[i], de2, dM0[i]); dM[i] = mul2(dM[i], rr2); }
                    else dM[i] = fma2(kk[i], de2, mul2(dM[i], rr2));
                }
                if (FROZEN && (tt0 + tl) % C == 0) {          // the chunk's first token: dM += dM0
#pragma unroll
                    for (int i = 0; i < 8; i++) { dM[i] = add2(dM[i], dM0[i]); dM0[i] = make_float2(0.f, 0.f); }
                }
                float ok[NOUT];
                ColReduce<TPR>::run(ck, lane, ok);
#pragma unroll
                for (int i = 0; i < NOUT; i++) pk[wcol + tl * D + i] = ok[i];
            }
            if (tl > 0) second_half(row - ROW, tl - 1);
        }
        // A tile shorter than the pipeline (only the sequence tail) has not yet waited for the
        // group that carries the next tile's streams.
        if (ntok < NST) cp_async_wait<0>();
        __syncthreads();
        // ── tile epilogue: cross-warp sums and coalesced stores ──
        for (int i = tid; i < ntok * D; i += NT) {
            float sq = 0.f, sk = 0.f;
#pragma unroll
            for (int w = 0; w < NW; w++) { sq += pq[(size_t)w * TB * D + i]; sk += pk[(size_t)w * TB * D + i]; }
            if (SPLIT > 1) {
                atomicAdd(&a.d_q[so + (size_t)tt0 * D + i], sq);
                atomicAdd(&a.d_k[so + (size_t)tt0 * D + i], sk);
            } else {
                a.d_q[so + (size_t)tt0 * D + i] = sq;
                a.d_k[so + (size_t)tt0 * D + i] = sk;
            }
        }
        for (int i = tid; i < ntok * ROWS; i += NT) {
            const int tl = i / ROWS, rr = i - tl * ROWS;
            a.d_v[so + (size_t)(tt0 + tl) * D + part * ROWS + rr] = dvs[i];
        }
        for (int job = warp; job < 3 * ntok; job += NW) {
            const int which = job / ntok, tl = job - which * ntok;
            float s = 0.f;
            for (int i = lane; i < ROWS; i += 32) s += scp[(which * TB + tl) * ROWS + i];
            s = warp_sum(s);
            if (lane == 0) {
                float* dst = (which == 0 ? a.d_alpha : which == 1 ? a.d_theta : a.d_eta) + go + tt0 + tl;
                const float val = (which == 2) ? s : -s;
                if (SPLIT > 1) atomicAdd(dst, val); else *dst = val;
            }
        }
        __syncthreads();   // partial rows are rewritten by the next tile
    }

    cp_async_wait<0>();
    if (a.atomic_out) {
        if (a.d_m_out == nullptr) return;   // batch-summed initial-state gradients not requested
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const size_t o = (size_t)r * D + col_of<D>((2 * i) ^ (xc << 2), cg);
            atomicAdd(&a.d_m_out[o], dM[i].x);
            atomicAdd(&a.d_m_out[o + 1], dM[i].y);
            atomicAdd(&a.d_s_out[o], dS[i].x);
            atomicAdd(&a.d_s_out[o + 1], dS[i].y);
        }
    } else if (a.d_m_out != nullptr) {
        store_state8<D>(dM, a.d_m_out + (size_t)b * DD, r, cg, xc);
        store_state8<D>(dS, a.d_s_out + (size_t)b * DD, r, cg, xc);
    }
}

template <int D>
static bool exact_bwd_launch(const BwdArgs& a, cudaStream_t st)
{
    if constexpr (D == 64) {
        if (split_rows(a.d, a.batch)) {
            // partial sums are added into these five outputs: start them from zero here
            const size_t nd = (size_t)a.batch * a.seq_len * D * sizeof(float), ng = (size_t)a.batch * a.seq_len * sizeof(float);
            cudaMemsetAsync(a.d_q, 0, nd, st); cudaMemsetAsync(a.d_k, 0, nd, st);
            cudaMemsetAsync(a.d_alpha, 0, ng, st); cudaMemsetAsync(a.d_theta, 0, ng, st); cudaMemsetAsync(a.d_eta, 0, ng, st);
            const size_t smem = exact_bwd_smem_floats<D, 2>() * sizeof(float);
            cudaFuncSetAttribute(titans_exact_bwd_kernel<D, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            titans_exact_bwd_kernel<D, 2><<<a.batch * 2, FastGeom<D, 2>::NT, smem, st>>>(a);
            return true;
        }
    }
    const size_t smem = exact_bwd_smem_floats<D>() * sizeof(float);
    cudaFuncSetAttribute(titans_exact_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    titans_exact_bwd_kernel<D><<<a.batch, FastGeom<D>::NT, smem, st>>>(a);
    return true;
}

// Frozen-M0 chunkwise Titans backward on a full M trajectory (a.m_traj [batch, seq_len + 1, d*d],
// a.chunk tokens per chunk, whole sequence).
template <int D>
static bool frozen_stream_bwd_launch(const BwdArgs& a, cudaStream_t st)
{
    const size_t smem = exact_bwd_smem_floats<D, 1, true>() * sizeof(float);
    cudaFuncSetAttribute(titans_exact_bwd_kernel<D, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    titans_exact_bwd_kernel<D, 1, true><<<a.batch, FastGeom<D>::NT, smem, st>>>(a);
    return true;
}

}  // namespace nlh
