// Frozen-M0 chunkwise Titans / Delta rule in CHUNK-PARALLEL (matrix) form, head dimension 64.
//
// Inside a frozen chunk the errors e_t = M0 k_t - v_t depend only on the chunk-start memory, so
// the whole chunk is linear in (M0, S0) with scalar gates and every product is a dense
// contraction over the chunk's tokens or over the head dimension — no per-token dependency
// chain is left inside a chunk; only the chunk boundaries form a sequential scan.
// With r_t = 1 - alpha_t and, for t >= j,
//     h(j,t)  = prod_{i=j+1..t} eta_i                     (decay of a momentum contribution)
//     Om(t,j) = r_t Om(t-1,j) + h(j,t),  Om(j,j) = 1      (weight of -theta_j e_j k_j^T in M_{t+1})
//     A_t = prod_{i<=t} r_i,  H_t = prod_{i<=t} eta_i,  B_t = r_t B_{t-1} + H_t   (weights of M0, S0)
// the forward of one chunk (rows = tokens) is
//     E   = K M0^T - V                        P = Q K^T
//     Y   = diag(A) Q M0^T + diag(B) Q S0^T - tril(W o P) E ,  W(t,j) = theta_j Om(t,j)
//     M_C = A_L M0 + B_L S0 - E^T diag(W(L-1,:)) K ,  S_C = H_L S0 - E^T diag(theta_j h(j,L-1)) K
// and the backward (G_M, G_S = gradients w.r.t. the chunk-end states, R = dY E^T) is
//     U   = tril(Om o P)^T dY + diag(Om(L-1,:)) K G_M^T + diag(h(:,L-1)) K G_S^T
//     dE  = -diag(theta) U,  dV = -dE,  dtheta_t = -<e_t, u_t>
//     dK  = -diag(theta)[ tril(Om o R)^T Q + diag(Om(L-1,:)) E G_M + diag(h(:,L-1)) E G_S ] + dE M0
//     dQ  = diag(A) dY M0 + diag(B) dY S0 - tril(W o R) K
//     G_M' = dY^T diag(A) Q + A_L G_M + dE^T K ,  G_S' = dY^T diag(B) Q + B_L G_M + H_L G_S
// plus the gate gradients d_alpha_t = -<M_t, lambda_t>, d_eta_t = <S_t, sigma_t>, which reduce to
// decayed scans over X = R o P (strictly lower triangle) and a few vectors (see the gate section).
// The Delta rule is the case eta = 0, S = 0. Same semantics as the per-token statement in
// core/kernels/titans_chunkwise_forward.cu:89-176 and titans_chunkwise_backward.cu:118-358
// (and the batched GEMM + phase-2 split of core/src/dispatch.rs:2608-2680, 2783-2878).
//
// One CTA of 256 threads per problem walks the chunks in order; every matrix of the chunk lives
// in shared memory as fp32 [64][68] (the padding makes both row- and column-wise 16-byte
// fragment loads bank-conflict free) and the contractions are FP32 FMA on 4x4 register tiles,
// so results agree with the per-token rule to rounding. The states never leave the chip between
// chunks and the k/v/q/dy streams are read exactly once.
#pragma once

#include "memory_fast.cuh"

namespace nlh {
namespace cmm {

constexpr int D = 64;            // head dimension
constexpr int CT = 64;           // tokens per chunk tile (chunk sizes up to 64)
constexpr int LD = 68;           // padded leading dimension of every shared-memory matrix
constexpr int SLOT = CT * LD;    // floats per matrix
constexpr int NT = 256;

// ── 4x4 register-tile fragments for thread (ty, tx) = (tid / 16, tid % 16) ──
// Output rows are always m = 4 ty + i. Output columns are n = 4 tx + j when B is stored [k][n]
// ("kn": n contiguous) and n = tx + 16 j when B is stored [n][k] ("nk": k contiguous).
__device__ __forceinline__ void lda_mk(float (&a)[4][4], const float* A, int ty, int k)
{
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float4 v = *reinterpret_cast<const float4*>(A + (4 * ty + i) * LD + k);
        a[i][0] = v.x; a[i][1] = v.y; a[i][2] = v.z; a[i][3] = v.w;
    }
}
__device__ __forceinline__ void lda_km(float (&a)[4][4], const float* A, int ty, int k)
{
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
        const float4 v = *reinterpret_cast<const float4*>(A + (k + kk) * LD + 4 * ty);
        a[0][kk] = v.x; a[1][kk] = v.y; a[2][kk] = v.z; a[3][kk] = v.w;
    }
}
__device__ __forceinline__ void ldb_kn(float (&b)[4][4], const float* B, int tx, int k)
{
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
        const float4 v = *reinterpret_cast<const float4*>(B + (k + kk) * LD + 4 * tx);
        b[kk][0] = v.x; b[kk][1] = v.y; b[kk][2] = v.z; b[kk][3] = v.w;
    }
}
__device__ __forceinline__ void ldb_nk(float (&b)[4][4], const float* B, int tx, int k)
{
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float4 v = *reinterpret_cast<const float4*>(B + (tx + 16 * j) * LD + k);
        b[0][j] = v.x; b[1][j] = v.y; b[2][j] = v.z; b[3][j] = v.w;
    }
}
__device__ __forceinline__ void fma44(float (&acc)[4][4], const float (&a)[4][4], const float (&b)[4][4])
{
#pragma unroll
    for (int kk = 0; kk < 4; kk++)
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i][kk], b[kk][j], acc[i][j]);
}
// a[i][kk] scaled by a per-row (i) factor / by a per-k (kk) factor
__device__ __forceinline__ void scale_rows(float (&o)[4][4], const float (&a)[4][4], const float (&s)[4])
{
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int kk = 0; kk < 4; kk++) o[i][kk] = a[i][kk] * s[i];
}
__device__ __forceinline__ void scale_k(float (&o)[4][4], const float (&a)[4][4], const float* s /*[4] at k*/)
{
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
        const float f = s[kk];
#pragma unroll
        for (int i = 0; i < 4; i++) o[i][kk] = a[i][kk] * f;
    }
}
__device__ __forceinline__ void scale_bk(float (&o)[4][4], const float (&b)[4][4], const float* s /*[4] at k*/)
{
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
        const float f = s[kk];
#pragma unroll
        for (int j = 0; j < 4; j++) o[kk][j] = b[kk][j] * f;
    }
}
__device__ __forceinline__ void zero44(float (&x)[4][4])
{
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) x[i][j] = 0.f;
}
// sum over the 16 tx lanes that share a ty (lanes 0-15 / 16-31 of a warp)
__device__ __forceinline__ float sum_tx(float v)
{
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    return v;
}

// Async copy of `rows` rows of 64 contiguous floats into a padded tile; rows [rows, CT) are zeroed.
__device__ __forceinline__ void tile_load(float* dst, const float* __restrict__ src, int rows)
{
    for (int p = threadIdx.x; p < CT * (D / 4); p += NT) {
        const int row = p >> 4, c4 = p & 15;
        float* d = dst + row * LD + c4 * 4;
        if (row < rows) cp_async16(d, src + (size_t)row * D + c4 * 4);
        else *reinterpret_cast<float4*>(d) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// per-chunk vectors in shared memory (64 floats each)
enum Vec { V_AL = 0, V_TH, V_ET, V_R, V_A, V_B, V_H, V_WM, V_WS, V_OM, V_OS, V_RE, V_ZM, V_ZS, V_GM, V_GS,
           V_T0, V_T1, V_T2, V_COUNT };
constexpr int SCAL = V_COUNT * CT;     // scalars follow the vectors
enum Scal { S_AT = 0, S_BT, S_HT, S_MM, S_SM, S_SS, S_COUNT = 8 };

constexpr size_t fwd_smem_bytes() { return ((size_t)10 * SLOT + 2 * 3 * CT + V_COUNT * CT + S_COUNT) * sizeof(float); }
constexpr size_t bwd_smem_bytes() { return ((size_t)13 * SLOT + V_COUNT * CT + S_COUNT + 32) * sizeof(float); }

// Gate-derived vectors of a chunk of L tokens (run by ONE thread; 64 short dependent steps):
// r, A, B, H and the totals at L-1; rho_end(t) = prod_{i=t+1..L-1} r_i.
template <int RULE>
__device__ __forceinline__ void chunk_vectors(float* vec, int L)
{
    float a = 1.f, b = 0.f, h = 1.f;
    for (int t = 0; t < CT; t++) {
        const float r = (t < L) ? 1.0f - vec[V_AL * CT + t] : 1.0f;
        const float e = (RULE == RULE_TITANS && t < L) ? vec[V_ET * CT + t] : 0.0f;
        vec[V_R * CT + t] = r;
        if (t < L) {
            a *= r;
            h *= e;
            b = fmaf(r, b, h);
        }
        vec[V_A * CT + t] = a; vec[V_B * CT + t] = b; vec[V_H * CT + t] = h;
    }
    vec[SCAL + S_AT] = a; vec[SCAL + S_BT] = b; vec[SCAL + S_HT] = h;
    float re = 1.f;
    for (int t = CT - 1; t >= 0; t--) {
        vec[V_RE * CT + t] = re;
        if (t < L && t > 0) re *= vec[V_R * CT + t];
        if (t >= L) re = 1.f;
    }
}

// ───────────────────────────────── forward ─────────────────────────────────
template <int RULE>
__global__ void __launch_bounds__(NT, 1) chunk_mm_fwd_kernel(FwdArgs a)
{
    constexpr bool HAS_S = (RULE == RULE_TITANS);
    extern __shared__ __align__(16) float sm[];
    float* Mb = sm;                       // M0 of the current chunk            [r][c]
    float* Sb = Mb + SLOT;                // S0                                  [r][c]
    float* Eb = Sb + SLOT;                // errors                              [t][r]
    float* Wb = Eb + SLOT;                // -W table, then -(W o P)             [t][s]
    float* KVQ = Wb + SLOT;               // [2][3] K | V (then the A,B part of y) | Q
    float* gat = KVQ + 6 * SLOT;          // [2][3][64] alpha | theta | eta
    float* vec = gat + 2 * 3 * CT;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int b = blockIdx.x;
    const int C = a.interval;
    const float* kg = a.k + (size_t)b * a.in_stride_tok * D;
    const float* vg = a.v + (size_t)b * a.in_stride_tok * D;
    const float* qg = a.q + (size_t)b * a.in_stride_tok * D;
    const float* alg = a.alpha + (size_t)b * a.in_stride_tok;
    const float* thg = a.theta + (size_t)b * a.in_stride_tok;
    const float* etg = HAS_S ? a.eta + (size_t)b * a.in_stride_tok : nullptr;
    float* yg = a.y + (size_t)b * a.seq_len * D;
    float* m_out = a.m_out + (size_t)b * a.out_stride;
    float* s_out = HAS_S ? a.s_out + (size_t)b * a.out_stride : nullptr;
    const int nc = (a.seq_len + C - 1) / C;

    auto prefetch = [&](int c) {
        const int t0 = c * C, L = min(C, a.seq_len - t0), buf = c & 1;
        float* base = KVQ + buf * 3 * SLOT;
        tile_load(base, kg + (size_t)t0 * D, L);
        tile_load(base + SLOT, vg + (size_t)t0 * D, L);
        tile_load(base + 2 * SLOT, qg + (size_t)t0 * D, L);
        if (tid < CT) {
            float* g = gat + buf * 3 * CT;
            if (tid < L) {
                cp_async4(g + tid, alg + t0 + tid);
                cp_async4(g + CT + tid, thg + t0 + tid);
                if (HAS_S) cp_async4(g + 2 * CT + tid, etg + t0 + tid);
            } else {
                g[tid] = 0.f; g[CT + tid] = 0.f; g[2 * CT + tid] = 0.f;
            }
        }
    };

    tile_load(Mb, a.m_init + (size_t)b * a.init_stride, D);
    if (HAS_S) tile_load(Sb, a.s_init + (size_t)b * a.init_stride, D);
    if (nc > 0) prefetch(0);
    cp_async_commit();

    for (int c = 0; c < nc; c++) {
        const int t0 = c * C, L = min(C, a.seq_len - t0), buf = c & 1;
        const int L4 = (L + 3) & ~3;
        float* Kb = KVQ + buf * 3 * SLOT;
        float* Vb = Kb + SLOT;
        float* Qb = Kb + 2 * SLOT;
        const float* g = gat + buf * 3 * CT;
        cp_async_wait<0>();
        __syncthreads();                     // chunk c staged; every thread is done with chunk c-1
        if (c + 1 < nc) prefetch(c + 1);
        cp_async_commit();
        if (c == 0) {                        // slot 0 = the initial state
            for (int p = tid; p < D * (D / 4); p += NT) {
                const int row = p >> 4, c4 = p & 15;
                *reinterpret_cast<float4*>(m_out + row * D + c4 * 4) = *reinterpret_cast<const float4*>(Mb + row * LD + c4 * 4);
                if (HAS_S) *reinterpret_cast<float4*>(s_out + row * D + c4 * 4) = *reinterpret_cast<const float4*>(Sb + row * LD + c4 * 4);
            }
        }
        // ── decay tables: column j of -W by thread j; gate vectors by thread 64 ──
        if (tid < CT) {
            const int j = tid;
            const float thj = g[CT + j];
            float om = 0.f, hh = 0.f, wm = 0.f, ws = 0.f;
            for (int t = 0; t < CT; t++) {
                if (t == j) { om = 1.f; hh = 1.f; }
                else if (t > j) {
                    hh *= HAS_S ? g[2 * CT + t] : 0.f;
                    om = fmaf(1.0f - g[t], om, hh);
                }
                const bool in = (t >= j) && (t < L) && (j < L);
                Wb[t * LD + j] = in ? -thj * om : 0.f;
                if (t == L - 1 && j < L) { wm = thj * om; ws = thj * hh; }
            }
            vec[V_WM * CT + j] = wm; vec[V_WS * CT + j] = ws;
        } else if (tid == CT) {
            for (int t = 0; t < CT; t++) {
                vec[V_AL * CT + t] = g[t];
                vec[V_ET * CT + t] = g[2 * CT + t];
            }
            chunk_vectors<RULE>(vec, L);
        }
        __syncthreads();

        // ── stage 1 (contraction over the head dimension): E, P, Q M0^T, Q S0^T ──
        {
            float accE[4][4], accP[4][4], accM[4][4], accS[4][4];
            zero44(accE); zero44(accP); zero44(accM); zero44(accS);
#pragma unroll 2
            for (int k = 0; k < D; k += 4) {
                float aK[4][4], aQ[4][4], bM[4][4], bK[4][4];
                lda_mk(aK, Kb, ty, k); lda_mk(aQ, Qb, ty, k);
                ldb_nk(bM, Mb, tx, k); ldb_nk(bK, Kb, tx, k);
                fma44(accE, aK, bM); fma44(accP, aQ, bK); fma44(accM, aQ, bM);
                if (HAS_S) { float bS[4][4]; ldb_nk(bS, Sb, tx, k); fma44(accS, aQ, bS); }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int t = 4 * ty + i;
                const float At = vec[V_A * CT + t], Bt = vec[V_B * CT + t];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int o = t * LD + tx + 16 * j;
                    Eb[o] = accE[i][j] - Vb[o];
                    Wb[o] *= accP[i][j];
                    Vb[o] = HAS_S ? fmaf(At, accM[i][j], Bt * accS[i][j]) : At * accM[i][j];
                }
            }
        }
        __syncthreads();

        // ── stage 2: y = A Q M0^T + B Q S0^T - tril(W o P) E  (contraction over earlier tokens) ──
        {
            float acc[4][4];
            zero44(acc);
            const int kend = min(L4, 4 * ty + 4);
            for (int k = 0; k < kend; k += 4) {
                float aw[4][4], be[4][4];
                lda_mk(aw, Wb, ty, k); ldb_kn(be, Eb, tx, k);
                fma44(acc, aw, be);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int t = 4 * ty + i;
                if (t < L) {
                    const float4 p = *reinterpret_cast<const float4*>(Vb + t * LD + 4 * tx);
                    *reinterpret_cast<float4*>(yg + (size_t)(t0 + t) * D + 4 * tx) =
                        make_float4(p.x + acc[i][0], p.y + acc[i][1], p.z + acc[i][2], p.w + acc[i][3]);
                }
            }
        }
        // ── stage 3: chunk-end states (contraction over the chunk's tokens) ──
        {
            float accM[4][4], accS[4][4];
            zero44(accM); zero44(accS);
            for (int k = 0; k < L4; k += 4) {
                float ae[4][4], bk[4][4], as[4][4];
                lda_km(ae, Eb, ty, k); ldb_kn(bk, Kb, tx, k);
                if (HAS_S) { scale_k(as, ae, vec + V_WS * CT + k); fma44(accS, as, bk); }
                scale_k(as, ae, vec + V_WM * CT + k);
                fma44(accM, as, bk);
            }
            const float At = vec[SCAL + S_AT], Bt = vec[SCAL + S_BT], Ht = vec[SCAL + S_HT];
            const size_t slot = (size_t)(c + 1) * D * D;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int o = (4 * ty + i) * LD + 4 * tx;
                const size_t go = slot + (size_t)(4 * ty + i) * D + 4 * tx;
                const float4 m = *reinterpret_cast<const float4*>(Mb + o);
                float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
                if (HAS_S) s = *reinterpret_cast<const float4*>(Sb + o);
                const float4 mn = make_float4(fmaf(At, m.x, fmaf(Bt, s.x, -accM[i][0])), fmaf(At, m.y, fmaf(Bt, s.y, -accM[i][1])),
                                              fmaf(At, m.z, fmaf(Bt, s.z, -accM[i][2])), fmaf(At, m.w, fmaf(Bt, s.w, -accM[i][3])));
                *reinterpret_cast<float4*>(Mb + o) = mn;
                *reinterpret_cast<float4*>(m_out + go) = mn;
                if (HAS_S) {
                    const float4 sn = make_float4(fmaf(Ht, s.x, -accS[i][0]), fmaf(Ht, s.y, -accS[i][1]),
                                                  fmaf(Ht, s.z, -accS[i][2]), fmaf(Ht, s.w, -accS[i][3]));
                    *reinterpret_cast<float4*>(Sb + o) = sn;
                    *reinterpret_cast<float4*>(s_out + go) = sn;
                }
            }
        }
    }
    if (nc == 0) {
        cp_async_wait<0>();
        __syncthreads();
        for (int p = tid; p < D * (D / 4); p += NT) {
            const int row = p >> 4, c4 = p & 15;
            *reinterpret_cast<float4*>(m_out + row * D + c4 * 4) = *reinterpret_cast<const float4*>(Mb + row * LD + c4 * 4);
            if (HAS_S) *reinterpret_cast<float4*>(s_out + row * D + c4 * 4) = *reinterpret_cast<const float4*>(Sb + row * LD + c4 * 4);
        }
    }
}

// ───────────────────────────────── backward ────────────────────────────────
// Chunks are walked last to first; G_M, G_S (gradients w.r.t. the chunk-end states) stay in
// shared memory. m_traj / s_traj hold the forward's chunk-boundary states (slot c = start of
// chunk c).
template <int RULE>
__global__ void __launch_bounds__(NT, 1) chunk_mm_bwd_kernel(BwdArgs a)
{
    constexpr bool HAS_S = (RULE == RULE_TITANS);
    extern __shared__ __align__(16) float sm[];
    float* GMb = sm;                      // d L / d M_C          [r][c]
    float* GSb = GMb + SLOT;              // d L / d S_C          [r][c]
    float* Kb = GSb + SLOT;               // [t][c]
    float* Qb = Kb + SLOT;                // [t][c]
    float* Yb = Qb + SLOT;                // dY [t][r]
    float* Mb = Yb + SLOT;                // M0 [r][c]
    float* Sb = Mb + SLOT;                // S0 [r][c]
    float* T6 = Sb + SLOT;                // V, then the boundary part of U        [t][r]
    float* Eb = T6 + SLOT;                // errors                                [t][r]
    float* T8 = Eb + SLOT;                // Om table [s][t], then dE              [t][r]
    float* T9 = T8 + SLOT;                // Om o P   [s][t], then the d_eta terms [t][j]
    float* T10 = T9 + SLOT;               // Om o R   [s][t]
    float* T11 = T10 + SLOT;              // X = R o P [s][t], then the d_alpha terms
    float* vec = T11 + SLOT;
    float* red = vec + V_COUNT * CT + S_COUNT;   // [32] block-reduction scratch
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x;
    const int C = a.chunk;
    const size_t so = (size_t)b * a.seq_len * D, go = (size_t)b * a.seq_len;
    const float* mtraj = a.m_traj + (size_t)b * a.traj_stride;
    const float* straj = HAS_S ? a.s_traj + (size_t)b * a.traj_stride : nullptr;
    const int nc = (a.seq_len + C - 1) / C;

    for (int p = tid; p < 2 * SLOT; p += NT) GMb[p] = 0.f;     // G_M = G_S = 0 beyond the sequence

    for (int c = nc - 1; c >= 0; c--) {
        const int t0 = c * C, L = min(C, a.seq_len - t0);
        const int L4 = (L + 3) & ~3;
        __syncthreads();                     // previous chunk fully consumed
        tile_load(Kb, a.k + so + (size_t)t0 * D, L);
        tile_load(Qb, a.q + so + (size_t)t0 * D, L);
        tile_load(Yb, a.d_y + so + (size_t)t0 * D, L);
        tile_load(T6, a.v + so + (size_t)t0 * D, L);
        tile_load(Mb, mtraj + (size_t)c * D * D, D);
        if (HAS_S) tile_load(Sb, straj + (size_t)c * D * D, D);
        if (tid < CT) {
            const bool in = tid < L;
            vec[V_AL * CT + tid] = in ? a.alpha[go + t0 + tid] : 0.f;
            vec[V_TH * CT + tid] = in ? a.theta[go + t0 + tid] : 0.f;
            vec[V_ET * CT + tid] = (in && HAS_S) ? a.eta[go + t0 + tid] : 0.f;
        }
        cp_async_commit();
        __syncthreads();                     // gates visible
        // ── tables: column t of Om(s,t) by thread t (overlaps the copies in flight) ──
        if (tid < CT) {
            const int j = tid;
            float om = 0.f, hh = 0.f, wm = 0.f, ws = 0.f;
            for (int t = 0; t < CT; t++) {
                if (t == j) { om = 1.f; hh = 1.f; }
                else if (t > j) {
                    hh *= vec[V_ET * CT + t];
                    om = fmaf(1.0f - vec[V_AL * CT + t], om, hh);
                }
                const bool in = (t >= j) && (t < L) && (j < L);
                T8[t * LD + j] = in ? om : 0.f;
                if (t == L - 1 && j < L) { wm = om; ws = hh; }
            }
            vec[V_OM * CT + j] = wm; vec[V_OS * CT + j] = ws;     // Om(L-1,j), h(j,L-1)
        } else if (tid == CT) {
            chunk_vectors<RULE>(vec, L);
        }
        cp_async_wait<0>();
        __syncthreads();

        // ── S1 (over the head dimension): E = K M0^T - V, P = Q K^T, K G_M^T, K G_S^T ──
        float accP[4][4];
        {
            float accE[4][4], accGM[4][4], accGS[4][4];
            zero44(accE); zero44(accP); zero44(accGM); zero44(accGS);
#pragma unroll 2
            for (int k = 0; k < D; k += 4) {
                float aK[4][4], aQ[4][4], bM[4][4], bK[4][4], bG[4][4];
                lda_mk(aK, Kb, ty, k); lda_mk(aQ, Qb, ty, k);
                ldb_nk(bM, Mb, tx, k); ldb_nk(bK, Kb, tx, k);
                fma44(accE, aK, bM); fma44(accP, aQ, bK);
                ldb_nk(bG, GMb, tx, k); fma44(accGM, aK, bG);
                if (HAS_S) { ldb_nk(bG, GSb, tx, k); fma44(accGS, aK, bG); }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int t = 4 * ty + i;
                const float om = vec[V_OM * CT + t], os = vec[V_OS * CT + t];
                float gm = 0.f, gs = 0.f;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int o = t * LD + tx + 16 * j;
                    const float e = accE[i][j] - T6[o];
                    Eb[o] = e;
                    gm = fmaf(e, accGM[i][j], gm);
                    if (HAS_S) gs = fmaf(e, accGS[i][j], gs);
                    T6[o] = HAS_S ? fmaf(om, accGM[i][j], os * accGS[i][j]) : om * accGM[i][j];
                }
                gm = sum_tx(gm);
                if (HAS_S) gs = sum_tx(gs);
                if (tx == 0) { vec[V_GM * CT + t] = gm; vec[V_GS * CT + t] = gs; }
            }
        }
        __syncthreads();
        // ── S2 (over the head dimension): R = dY E^T; weighted tables Om o P, Om o R, X = R o P ──
        {
            float accR[4][4];
            zero44(accR);
#pragma unroll 2
            for (int k = 0; k < D; k += 4) {
                float aY[4][4], bE[4][4];
                lda_mk(aY, Yb, ty, k); ldb_nk(bE, Eb, tx, k);
                fma44(accR, aY, bE);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int s = 4 * ty + i;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int t = tx + 16 * j, o = s * LD + t;
                    const float om = T8[o];
                    T9[o] = om * accP[i][j];
                    T10[o] = om * accR[i][j];
                    T11[o] = (s > t && s < L) ? accR[i][j] * accP[i][j] : 0.f;
                }
            }
        }
        __syncthreads();
        // ── S3 (over the chunk's tokens): U, the token part of dK (Z) and of dQ ──
        float accZ[4][4], accQ[4][4];
        {
            float accU[4][4];
            zero44(accU); zero44(accZ); zero44(accQ);
            for (int k = 4 * ty; k < L4; k += 4) {            // rows t = 4ty.. need s >= t
                float aP[4][4], aR[4][4], bY[4][4], bQ[4][4];
                lda_km(aP, T9, ty, k); ldb_kn(bY, Yb, tx, k); fma44(accU, aP, bY);
                lda_km(aR, T10, ty, k); ldb_kn(bQ, Qb, tx, k); fma44(accZ, aR, bQ);
            }
            const int kend = min(L4, 4 * ty + 4);              // rows s = 4ty.. need t <= s
            for (int k = 0; k < kend; k += 4) {
                float aR[4][4], bK[4][4], bT[4][4];
                lda_mk(aR, T10, ty, k); ldb_kn(bK, Kb, tx, k);
                scale_bk(bT, bK, vec + V_TH * CT + k);
                fma44(accQ, aR, bT);
            }
            // (the Om table in T8 was last read before the barrier above: dE may replace it)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int t = 4 * ty + i, o = t * LD + 4 * tx;
                const float th = vec[V_TH * CT + t];
                const float4 ub = *reinterpret_cast<const float4*>(T6 + o);
                const float4 e = *reinterpret_cast<const float4*>(Eb + o);
                const float u0 = accU[i][0] + ub.x, u1 = accU[i][1] + ub.y, u2 = accU[i][2] + ub.z, u3 = accU[i][3] + ub.w;
                *reinterpret_cast<float4*>(T8 + o) = make_float4(-th * u0, -th * u1, -th * u2, -th * u3);   // dE
                if (t < L)
                    *reinterpret_cast<float4*>(a.d_v + so + (size_t)(t0 + t) * D + 4 * tx) =
                        make_float4(th * u0, th * u1, th * u2, th * u3);
                float dt = fmaf(e.x, u0, fmaf(e.y, u1, fmaf(e.z, u2, e.w * u3)));
                dt = sum_tx(dt);
                if (tx == 0 && t < L) a.d_theta[go + t0 + t] = -dt;
#pragma unroll
                for (int j = 0; j < 4; j++) accQ[i][j] = -accQ[i][j];
            }
        }
        __syncthreads();
        // ── S4a (over the head dimension): Z += Om(L-1,t) E G_M + h(t,L-1) E G_S ──
        {
            float om[4], os[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { om[i] = vec[V_OM * CT + 4 * ty + i]; os[i] = vec[V_OS * CT + 4 * ty + i]; }
#pragma unroll 2
            for (int k = 0; k < D; k += 4) {
                float aE[4][4], aS[4][4], bG[4][4];
                lda_mk(aE, Eb, ty, k);
                ldb_kn(bG, GMb, tx, k); scale_rows(aS, aE, om); fma44(accZ, aS, bG);
                if (HAS_S) { ldb_kn(bG, GSb, tx, k); scale_rows(aS, aE, os); fma44(accZ, aS, bG); }
            }
        }
        // ── S4b (over the head dimension): dK = -theta Z + dE M0; dQ += A dY M0 + B dY S0 ──
        {
            float accK[4][4], accDM[4][4], accDS[4][4];
            zero44(accK); zero44(accDM); zero44(accDS);
#pragma unroll 2
            for (int k = 0; k < D; k += 4) {
                float aD[4][4], aY[4][4], bM[4][4];
                lda_mk(aD, T8, ty, k); lda_mk(aY, Yb, ty, k); ldb_kn(bM, Mb, tx, k);
                fma44(accK, aD, bM); fma44(accDM, aY, bM);
                if (HAS_S) { float bS[4][4]; ldb_kn(bS, Sb, tx, k); fma44(accDS, aY, bS); }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int t = 4 * ty + i, o = t * LD + 4 * tx;
                const float th = vec[V_TH * CT + t], At = vec[V_A * CT + t], Bt = vec[V_B * CT + t];
                const float4 qv = *reinterpret_cast<const float4*>(Qb + o);
                float zm = fmaf(qv.x, accDM[i][0], fmaf(qv.y, accDM[i][1], fmaf(qv.z, accDM[i][2], qv.w * accDM[i][3])));
                float zs = 0.f;
                if (HAS_S) zs = fmaf(qv.x, accDS[i][0], fmaf(qv.y, accDS[i][1], fmaf(qv.z, accDS[i][2], qv.w * accDS[i][3])));
                zm = sum_tx(zm);
                if (HAS_S) zs = sum_tx(zs);
                if (tx == 0) { vec[V_ZM * CT + t] = zm; vec[V_ZS * CT + t] = zs; }
                if (t < L) {
                    const size_t g4 = so + (size_t)(t0 + t) * D + 4 * tx;
                    *reinterpret_cast<float4*>(a.d_k + g4) =
                        make_float4(fmaf(-th, accZ[i][0], accK[i][0]), fmaf(-th, accZ[i][1], accK[i][1]),
                                    fmaf(-th, accZ[i][2], accK[i][2]), fmaf(-th, accZ[i][3], accK[i][3]));
                    float qo[4];
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        qo[j] = accQ[i][j] + At * accDM[i][j] + (HAS_S ? Bt * accDS[i][j] : 0.f);
                    *reinterpret_cast<float4*>(a.d_q + g4) = make_float4(qo[0], qo[1], qo[2], qo[3]);
                }
            }
        }
        // ── Frobenius products <M0,G_M>, <S0,G_M>, <S0,G_S> (before G is replaced) ──
        {
            float pm = 0.f, ps = 0.f, pss = 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int o = (4 * ty + i) * LD + 4 * tx;
                const float4 m = *reinterpret_cast<const float4*>(Mb + o);
                const float4 g = *reinterpret_cast<const float4*>(GMb + o);
                pm += m.x * g.x + m.y * g.y + m.z * g.z + m.w * g.w;
                if (HAS_S) {
                    const float4 s = *reinterpret_cast<const float4*>(Sb + o);
                    const float4 gs = *reinterpret_cast<const float4*>(GSb + o);
                    ps += s.x * g.x + s.y * g.y + s.z * g.z + s.w * g.w;
                    pss += s.x * gs.x + s.y * gs.y + s.z * gs.z + s.w * gs.w;
                }
            }
            pm = warp_sum(pm); ps = warp_sum(ps); pss = warp_sum(pss);
            if (lane == 0) { red[warp] = pm; red[8 + warp] = ps; red[16 + warp] = pss; }
        }
        // ── S5 (over the chunk's tokens): chunk-start gradients G_M', G_S' ──
        {
            float accM[4][4], accS[4][4];
            zero44(accM); zero44(accS);
            for (int k = 0; k < L4; k += 4) {
                float aY[4][4], aD[4][4], bQ[4][4], bK[4][4], bT[4][4];
                lda_km(aY, Yb, ty, k); ldb_kn(bQ, Qb, tx, k);
                scale_bk(bT, bQ, vec + V_A * CT + k); fma44(accM, aY, bT);
                if (HAS_S) { scale_bk(bT, bQ, vec + V_B * CT + k); fma44(accS, aY, bT); }
                lda_km(aD, T8, ty, k); ldb_kn(bK, Kb, tx, k); fma44(accM, aD, bK);
            }
            __syncthreads();                                   // every read of G_M, G_S above is done
            const float At = vec[SCAL + S_AT], Bt = vec[SCAL + S_BT], Ht = vec[SCAL + S_HT];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int o = (4 * ty + i) * LD + 4 * tx;
                const float4 g = *reinterpret_cast<const float4*>(GMb + o);
                *reinterpret_cast<float4*>(GMb + o) = make_float4(fmaf(At, g.x, accM[i][0]), fmaf(At, g.y, accM[i][1]),
                                                                  fmaf(At, g.z, accM[i][2]), fmaf(At, g.w, accM[i][3]));
                if (HAS_S) {
                    const float4 gs = *reinterpret_cast<const float4*>(GSb + o);
                    *reinterpret_cast<float4*>(GSb + o) =
                        make_float4(fmaf(Bt, g.x, fmaf(Ht, gs.x, accS[i][0])), fmaf(Bt, g.y, fmaf(Ht, gs.y, accS[i][1])),
                                    fmaf(Bt, g.z, fmaf(Ht, gs.z, accS[i][2])), fmaf(Bt, g.w, fmaf(Ht, gs.w, accS[i][3])));
                }
            }
        }
        // ── gate gradients. With XX_t[j] = sum_{s>=t} rho(t,s) X[s,j], YY_t[j] = XX_t[j] + eta_{t+1} YY_{t+1}[j]
        //    (and the same two scans ZM, ZS / ZSs over the vectors zM, zS):
        //    <M_t,lambda_t> = A_{t-1} ZM_t + B_{t-1} ZS_t + rho(t,L-1)(A_{t-1} mm + B_{t-1} sm)
        //                     - sum_{j<t} theta_j Om(t-1,j) (XX_t[j] + rho(t,L-1) gM_j)
        //    <S_t,sigma_t>  = H_{t-1} (ZSs_t + Om(L-1,t) sm + h(t,L-1) ss)
        //                     - sum_{j<t} theta_j h(j,t-1) (YY_t[j] + Om(L-1,t) gM_j + h(t,L-1) gS_j)
        if (tid < CT) {
            const int j = tid;
            if (j < L) {
                float xx = 0.f, yy = 0.f;
                for (int t = L - 1; t > j; t--) {              // reverse scans down column j
                    const float rn = (t + 1 < L) ? vec[V_R * CT + t + 1] : 0.f;
                    const float en = (t + 1 < L) ? vec[V_ET * CT + t + 1] : 0.f;
                    xx = fmaf(rn, xx, T11[t * LD + j]);
                    yy = fmaf(en, yy, xx);
                    T11[t * LD + j] = xx;
                    T9[t * LD + j] = yy;
                }
                const float thj = vec[V_TH * CT + j], gm = vec[V_GM * CT + j], gs = vec[V_GS * CT + j];
                float om = 1.f, hh = 1.f;                      // Om(t-1,j), h(j,t-1) at t = j+1
                for (int t = j + 1; t < L; t++) {
                    const float re = vec[V_RE * CT + t], omL = vec[V_OM * CT + t], osL = vec[V_OS * CT + t];
                    T11[t * LD + j] = thj * om * fmaf(re, gm, T11[t * LD + j]);
                    T9[t * LD + j] = thj * hh * (T9[t * LD + j] + omL * gm + osL * gs);
                    hh *= vec[V_ET * CT + t];
                    om = fmaf(vec[V_R * CT + t], om, hh);
                }
            }
        } else if (tid == CT) {                                // scans over the vectors zM, zS
            float zm = 0.f, zs = 0.f, zss = 0.f;
            for (int t = L - 1; t >= 0; t--) {
                const float rn = (t + 1 < L) ? vec[V_R * CT + t + 1] : 0.f;
                const float en = (t + 1 < L) ? vec[V_ET * CT + t + 1] : 0.f;
                zm = fmaf(rn, zm, vec[V_ZM * CT + t]);
                zs = fmaf(rn, zs, vec[V_ZS * CT + t]);
                zss = fmaf(en, zss, zs);
                vec[V_T0 * CT + t] = zm; vec[V_T1 * CT + t] = zs; vec[V_T2 * CT + t] = zss;
            }
        } else if (tid == CT + 32) {                           // finish the Frobenius products
            float pm = 0.f, ps = 0.f, pss = 0.f;
            for (int w = 0; w < 8; w++) { pm += red[w]; ps += red[8 + w]; pss += red[16 + w]; }
            vec[SCAL + S_MM] = pm; vec[SCAL + S_SM] = ps; vec[SCAL + S_SS] = pss;
        }
        __syncthreads();
        if (tid < L) {
            const int t = tid;
            float sa = 0.f, se = 0.f;
            for (int j4 = 0; j4 < t; j4 += 4) {
                const float4 x = *reinterpret_cast<const float4*>(T11 + t * LD + j4);
                const float4 y = *reinterpret_cast<const float4*>(T9 + t * LD + j4);
                sa += x.x; se += y.x;
                if (j4 + 1 < t) { sa += x.y; se += y.y; }
                if (j4 + 2 < t) { sa += x.z; se += y.z; }
                if (j4 + 3 < t) { sa += x.w; se += y.w; }
            }
            const float Am = t > 0 ? vec[V_A * CT + t - 1] : 1.f;
            const float Bm = t > 0 ? vec[V_B * CT + t - 1] : 0.f;
            const float Hm = t > 0 ? vec[V_H * CT + t - 1] : 1.f;
            const float mm = vec[SCAL + S_MM], smv = vec[SCAL + S_SM], ssv = vec[SCAL + S_SS];
            const float re = vec[V_RE * CT + t];
            const float da = Am * vec[V_T0 * CT + t] + Bm * vec[V_T1 * CT + t] + re * (Am * mm + Bm * smv) - sa;
            a.d_alpha[go + t0 + t] = -da;
            if (HAS_S) {
                const float de = Hm * (vec[V_T2 * CT + t] + vec[V_OM * CT + t] * smv + vec[V_OS * CT + t] * ssv) - se;
                a.d_eta[go + t0 + t] = de;
            }
        }
    }
    __syncthreads();
    // d_m_initial / d_s_initial: summed over the batch (drop-in entries) or per problem; not
    // written at all when the caller passed NULL
    if (a.d_m_out == nullptr) return;
    for (int p = tid; p < D * D; p += NT) {
        const int row = p >> 6, col = p & 63;
        const float gm = GMb[row * LD + col];
        if (a.atomic_out) atomicAdd(&a.d_m_out[p], gm);
        else a.d_m_out[(size_t)b * D * D + p] = gm;
        if (HAS_S) {
            const float gs = GSb[row * LD + col];
            if (a.atomic_out) atomicAdd(&a.d_s_out[p], gs);
            else a.d_s_out[(size_t)b * D * D + p] = gs;
        }
    }
}

// ───────────────────────────── host dispatch ─────────────────────────────
// Chunk sizes below this run the per-token register kernels (a 64-token tile would be mostly
// padding).
constexpr int MIN_CHUNK = 16;

inline bool shape_ok(int d, int chunk, float clip, float mmax)
{
    return d == D && chunk >= MIN_CHUNK && chunk <= CT && !(clip > 0.0f) && !m_norm_enabled(mmax);
}

static bool forward(int rule, const FwdArgs& a, cudaStream_t st)
{
    if (!a.frozen || a.store_mode != STORE_CHUNK || !shape_ok(a.d, a.interval, a.error_clip, a.m_norm_max)) return false;
    if (rule != RULE_TITANS && rule != RULE_DELTA) return false;
    const bool al = aligned16(a.k) && aligned16(a.v) && aligned16(a.q) && aligned16(a.y) && aligned16(a.m_init) &&
                    aligned16(a.m_out) && (rule != RULE_TITANS || (a.s_init && a.s_out && aligned16(a.s_init) && aligned16(a.s_out))) &&
                    (a.init_stride % 4 == 0) && (a.out_stride % 4 == 0);
    if (!al) return false;
    const int smem = (int)fwd_smem_bytes();
    if (rule == RULE_TITANS) {
        cudaFuncSetAttribute(chunk_mm_fwd_kernel<RULE_TITANS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        chunk_mm_fwd_kernel<RULE_TITANS><<<a.batch, NT, smem, st>>>(a);
    } else {
        cudaFuncSetAttribute(chunk_mm_fwd_kernel<RULE_DELTA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        chunk_mm_fwd_kernel<RULE_DELTA><<<a.batch, NT, smem, st>>>(a);
    }
    return true;
}

static bool backward(int rule, const BwdArgs& a, cudaStream_t st)
{
    if (!a.frozen || !shape_ok(a.d, a.chunk, a.error_clip, a.m_norm_max)) return false;
    if (rule != RULE_TITANS && rule != RULE_DELTA) return false;
    if (a.d_m_seed != nullptr || a.d_s_seed != nullptr) return false;
    const bool al = aligned16(a.k) && aligned16(a.v) && aligned16(a.q) && aligned16(a.d_y) && aligned16(a.d_k) &&
                    aligned16(a.d_v) && aligned16(a.d_q) && aligned16(a.m_traj) && (a.traj_stride % 4 == 0) &&
                    (rule != RULE_TITANS || (a.s_traj && aligned16(a.s_traj)));
    if (!al) return false;
    const int smem = (int)bwd_smem_bytes();
    if (rule == RULE_TITANS) {
        cudaFuncSetAttribute(chunk_mm_bwd_kernel<RULE_TITANS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        chunk_mm_bwd_kernel<RULE_TITANS><<<a.batch, NT, smem, st>>>(a);
    } else {
        cudaFuncSetAttribute(chunk_mm_bwd_kernel<RULE_DELTA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        chunk_mm_bwd_kernel<RULE_DELTA><<<a.batch, NT, smem, st>>>(a);
    }
    return true;
}

}  // namespace cmm
}  // namespace nlh
