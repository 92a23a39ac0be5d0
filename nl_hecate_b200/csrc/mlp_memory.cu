// Titans LMM with a two-layer MLP memory (deep neural memory): forward / backward kernel pair.
// Replaces titans_mlp_forward_f32_cuda / titans_mlp_backward_f32_cuda of the reference
// (core/src/cuda_ffi.rs:854-911, kernels core/kernels/titans_mlp_forward.cu:112-330 and
// titans_mlp_backward.cu:99-562; CPU statement TitansLMM::step_mlp / step_backward_mlp,
// core/src/titans_lmm.rs:653-1131).
//
// Memory state: M = {W1[dh,d], b1[dh], W2[d,dh], b2[d]} packed flat (ss floats); S the same shape.
//   token t:  pre = W1 k + b1, h = act(pre), e = W2 h + b2 - v, gp = (W2^T e) * act'(pre)
//             grad = {gp k^T, gp, e h^T, e};  S' = eta S - theta grad;  M' = (1-alpha) M + S'
//             (optional Frobenius projection of M');  y = MLP(M', q)
//
// Layout on the SM, one CTA of 512 threads per problem (problems are independent):
//   forward   M lives in shared memory (the four matrix-vector products of a token read it there),
//             S lives in registers (it is only touched element-wise); both are written once per
//             token to the caller's trajectories with coalesced stores — the 2 x ss x 4 bytes per
//             token the ABI asks for, which is what bounds the kernel (HBM writes).
//   backward  dM lives in registers (element-wise only), dS in shared memory (the second-order
//             terms are matrix-vector products with dS); M_t, M_{t+1}, S_t are read from the stored
//             trajectories. M_{t+1} of token t is M_t of token t+1's predecessor, so every state
//             comes from HBM once and from L2 afterwards.
// The reference keeps all of this in global memory with 8-10 block barriers and serial loops per
// token; the arithmetic here is the same, the order of the sums is not (fp32, relative 1e-5).
#include "nlh_common.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {
namespace mlpm {

constexpr int NT = 512;
constexpr int NW = NT / 32;
enum { ACT_GELU = 0, ACT_SILU = 1, ACT_RELU = 2 };

struct Dims {
    int d, dh;
    int o1, o2, o3, ss;      // offsets of b1, W2, b2 in the packed state; its size
    int tps_d, tps_h;        // log2 of the threads that share a row of d / dh columns (32 each)
    FastDiv div_d, div_h;
};

static Dims make_dims(int d, int dh)
{
    Dims D;
    D.d = d; D.dh = dh;
    D.o1 = dh * d; D.o2 = D.o1 + dh; D.o3 = D.o2 + d * dh; D.ss = D.o3 + d;
    D.div_d = make_fastdiv(d); D.div_h = make_fastdiv(dh);
    D.tps_d = 0; while ((32 << D.tps_d) < d) D.tps_d++;
    D.tps_h = 0; while ((32 << D.tps_h) < dh) D.tps_h++;
    return D;
}

template <int ACT> __device__ __forceinline__ float act_fn(float x)
{
    if (ACT == ACT_GELU) {
        const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
        return 0.5f * x * (1.0f + tanhf(inner));
    }
    if (ACT == ACT_SILU) return x / (1.0f + expf(-x));
    return fmaxf(x, 0.0f);
}
template <int ACT> __device__ __forceinline__ float act_prime(float x)
{
    if (ACT == ACT_GELU) {
        const float c = 0.7978845608028654f, a = 0.044715f;
        const float t = tanhf(c * (x + a * x * x * x));
        return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * c * (1.0f + 3.0f * a * x * x);
    }
    if (ACT == ACT_SILU) {
        const float s = 1.0f / (1.0f + expf(-x));
        return s * (1.0f + x * (1.0f - s));
    }
    return x > 0.0f ? 1.0f : 0.0f;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Shared-memory layout: one pad float after every 32, for matrices (the whole packed state keeps
// its flat order) and vectors alike. A thread that walks 32 consecutive columns of its own row then
// hits 32 different banks whatever the row length, threads on consecutive elements still do, and
// a vector read at 32 p + j by threads with different p does too.
__device__ __forceinline__ int P(int i) { return i + (i >> 5); }
__host__ __device__ inline int padded(int n) { return n + (n >> 5) + 1; }

// out(r) = sum_c W[r, c] x[c], r < R: W row-major [R, C] at flat offset off of the padded buffer
// Wp, x a padded vector. 2^tps threads per row, each a 32-column segment, combined by shuffles;
// every (row, segment) pair of the matrix is in flight at once (R * 2^tps <= NT for the sizes of the
// reference's configs), so a product is one pass of 32 FMAs instead of a chain of row iterations.
// epi(r, sum) runs on one thread per row.
template <class Epi>
__device__ __forceinline__ void rowdot(const float* Wp, int off, int R, int C, int tps, const float* xp, Epi epi)
{
    const int TP = 1 << tps, T = (C + 31) >> 5;
    for (int u0 = 0; u0 < (R << tps); u0 += NT) {
        const int u = u0 + threadIdx.x, r = u >> tps, p = u & (TP - 1);
        float acc = 0.0f;
        if (r < R && p < T) {
            const int c0 = p << 5, n = min(32, C - c0), f0 = off + r * C + c0;
            const float* xs = xp + c0 + p;
            if ((f0 & 31) == 0 && n == 32) {
                const float* w = Wp + f0 + (f0 >> 5);
                float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    a0 = fmaf(w[j], xs[j], a0); a1 = fmaf(w[j + 1], xs[j + 1], a1);
                    a2 = fmaf(w[j + 2], xs[j + 2], a2); a3 = fmaf(w[j + 3], xs[j + 3], a3);
                }
                acc = (a0 + a1) + (a2 + a3);
            } else {
                for (int j = 0; j < n; j++) acc = fmaf(Wp[P(f0 + j)], xs[j], acc);
            }
        }
        for (int o = TP >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (r < R && p == 0) epi(r, acc);
    }
}

// out(j) = sum_i W[i, j] x[i] for j < C (C <= NT), W at flat offset off of a padded shared buffer
// (PAD) or of global memory. Thread (g, j) adds rows g, g + G, ...; the G partial sums meet in
// scr[NT]; epi(j, sum) runs on threads j < C. Two block barriers inside: every thread must call it.
template <bool PAD, class Epi>
__device__ __forceinline__ void colsum(const float* __restrict__ W, int off, int R, int C, const float* xp, float* scr,
                                       int g, int j, int G, Epi epi)
{
    float acc = 0.0f;
    if (g < G) {
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        int i = g;
        for (; i + 3 * G < R; i += 4 * G) {
            const int f0 = off + i * C + j, f1 = f0 + G * C, f2 = f1 + G * C, f3 = f2 + G * C;
            const float w0 = W[PAD ? P(f0) : f0], w1 = W[PAD ? P(f1) : f1], w2 = W[PAD ? P(f2) : f2], w3 = W[PAD ? P(f3) : f3];
            a0 = fmaf(w0, xp[P(i)], a0); a1 = fmaf(w1, xp[P(i + G)], a1);
            a2 = fmaf(w2, xp[P(i + 2 * G)], a2); a3 = fmaf(w3, xp[P(i + 3 * G)], a3);
        }
        for (; i < R; i += G) { const int f = off + i * C + j; a0 = fmaf(W[PAD ? P(f) : f], xp[P(i)], a0); }
        acc = (a0 + a1) + (a2 + a3);
        scr[g * C + j] = acc;
    }
    __syncthreads();
    if ((int)threadIdx.x < C) {
        float s = 0.0f;
        for (int gg = 0; gg < G; gg++) s += scr[gg * C + threadIdx.x];
        epi((int)threadIdx.x, s);
    }
    __syncthreads();
}

// Sum of K per-thread values over the CTA; the result is valid on every thread. red: K * NW floats.
template <int K>
__device__ __forceinline__ void block_sum(float (&v)[K], float* red)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int q = 0; q < K; q++) {
        const float s = warp_sum(v[q]);
        if (lane == 0) red[q * NW + warp] = s;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < K; q++) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; w++) s += red[q * NW + w];
        v[q] = s;
    }
    __syncthreads();
}

// Element idx of the packed state -> outer-product term built from four padded vectors:
//   W1[r,c] -> a1[r] * x1[c],  b1[r] -> a1[r],  W2[r,c] -> a2[r] * x2[c],  b2[r] -> a2[r]
// SD, SDH != 0: the sizes are compile-time constants that divide NT, so for the elements
// idx = tid + i * NT of one thread the column of W1 is always tid % SD and the column of W2 always
// tid % SDH; x1c = x1[tid % SD] and x2c = x2[tid % SDH] are then loaded once per pass by the caller,
// and the region tests and row numbers fold to constants and shifts in the unrolled loops.
template <int SD, int SDH>
__device__ __forceinline__ float outer_term(const Dims& D, int idx, const float* a1, const float* x1, float x1c,
                                            const float* a2, const float* x2, float x2c)
{
    if (SD != 0) {
        constexpr int o1 = SDH * SD, o2 = o1 + SDH, o3 = o2 + SD * SDH;
        if (idx < o1) return a1[P(idx / (SD ? SD : 1))] * x1c;
        if (idx < o2) return a1[P(idx - o1)];
        if (idx < o3) return a2[P((idx - o2) / (SDH ? SDH : 1))] * x2c;
        return a2[P(idx - o3)];
    }
    if (idx < D.o1) { const int r = fd_div(idx, D.div_d); return a1[P(r)] * x1[P(idx - r * D.d)]; }
    if (idx < D.o2) return a1[P(idx - D.o1)];
    if (idx < D.o3) { const int e = idx - D.o2; const int r = fd_div(e, D.div_h); return a2[P(r)] * x2[P(e - r * D.dh)]; }
    return a2[P(idx - D.o3)];
}
constexpr int PNT = NT + NT / 32;      // padded distance of two elements NT apart
constexpr int UB = 8;                  // elements whose loads are issued before their stores

// n consecutive floats of global memory into a padded shared buffer (coalesced, 8 loads in flight)
__device__ __forceinline__ void stage(float* dstp, const float* __restrict__ src, int n)
{
    int f = threadIdx.x;
    for (; f + 7 * NT < n; f += 8 * NT) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = src[f + u * NT];
#pragma unroll
        for (int u = 0; u < 8; u++) dstp[P(f + u * NT)] = v[u];
    }
    for (; f < n; f += NT) dstp[P(f)] = src[f];
}

struct FwdArgs {
    const float *k, *v, *q, *alpha, *theta, *eta, *m_init, *s_init;
    float *m_states, *s_states, *y;
    int seq_len;
    long long in_stride, m_stride;
    float m_norm_max;
    Dims D;
};

inline size_t fwd_smem_floats(const Dims& D) { return (size_t)padded(D.ss) + 4 * padded(D.d) + 3 * padded(D.dh) + NT + 4 * NW; }

template <int ACT, int EPT, int SD, int SDH>
__global__ void __launch_bounds__(NT, 1) mlp_fwd_kernel(FwdArgs a)
{
    extern __shared__ __align__(16) float sm[];
    const Dims& D = a.D;
    const int d = SD ? SD : D.d, dh = SD ? SDH : D.dh, ss = SD ? 2 * SD * SDH + SD + SDH : D.ss;
    const int tid = threadIdx.x, b = blockIdx.x, ptid = P(tid);
    __builtin_assume(tid >= 0 && tid < NT);
    const int pd = padded(d), ph = padded(dh);
    float* Msm = sm;                       // the packed state, padded
    float* kb = Msm + padded(ss);
    float* vb = kb + pd;
    float* qb = vb + pd;
    float* e = qb + pd;
    float* pre = e + pd;
    float* h = pre + ph;
    float* gp = h + ph;
    float* scr = gp + ph;
    float* red = scr + NT;

    const float* k = a.k + (size_t)b * a.in_stride;
    const float* v = a.v + (size_t)b * a.in_stride;
    const float* q = a.q + (size_t)b * a.in_stride;
    float* y = a.y + (size_t)b * a.in_stride;
    const float* alpha = a.alpha + (size_t)b * a.seq_len;
    const float* theta = a.theta + (size_t)b * a.seq_len;
    const float* eta = a.eta + (size_t)b * a.seq_len;
    float* mt = a.m_states + (size_t)b * a.m_stride;
    float* st = a.s_states + (size_t)b * a.m_stride;
    const bool clamp = m_norm_enabled(a.m_norm_max);
    const int gh_ = fd_div(tid, D.div_h), jh = tid - gh_ * dh, Gh = NT / dh;   // column split for C = dh

    float S[EPT];
#pragma unroll
    for (int i = 0; i < EPT; i++) {
        const int idx = tid + i * NT;
        S[i] = 0.0f;
        if (idx < ss) {
            const float m = a.m_init[(size_t)b * ss + idx];
            S[i] = a.s_init[(size_t)b * ss + idx];
            Msm[ptid + i * PNT] = m; mt[idx] = m; st[idx] = S[i];
        }
    }
    for (int t = 0; t < a.seq_len; t++) {
        for (int i = tid; i < 3 * d; i += NT) {
            const int w = fd_div(i, D.div_d), c = i - w * d;
            (w == 0 ? kb : w == 1 ? vb : qb)[P(c)] = (w == 0 ? k : w == 1 ? v : q)[(size_t)t * d + c];
        }
        const float al = alpha[t], th = theta[t], et = eta[t];
        __syncthreads();
        rowdot(Msm, 0, dh, d, D.tps_d, kb, [&](int r, float s) { const float p = s + Msm[P(D.o1 + r)]; pre[P(r)] = p; h[P(r)] = act_fn<ACT>(p); });
        __syncthreads();
        rowdot(Msm, D.o2, d, dh, D.tps_h, h, [&](int r, float s) { e[P(r)] = s + Msm[P(D.o3 + r)] - vb[P(r)]; });
        __syncthreads();
        colsum<true>(Msm, D.o2, d, dh, e, scr, gh_, jh, Gh, [&](int j, float s) { gp[P(j)] = s * act_prime<ACT>(pre[P(j)]); });
        // S' = eta S - theta grad, M' = (1 - alpha) M + S'
        float* mn = mt + (size_t)(t + 1) * ss;
        float* sn = st + (size_t)(t + 1) * ss;
        float sq[1] = {0.0f};
        const float keep = 1.0f - al;
        const float x1c = SD ? kb[P(tid % (SD ? SD : 1))] : 0.0f, x2c = SD ? h[P(tid % (SDH ? SDH : 1))] : 0.0f;
#pragma unroll
        for (int i0 = 0; i0 < EPT; i0 += UB) {
            float g[UB], mo[UB];
#pragma unroll
            for (int u = 0; u < UB; u++) {
                const int i = i0 + u, idx = tid + i * NT;
                if (i < EPT && idx < ss) {
                    g[u] = outer_term<SD, SDH>(D, idx, gp, kb, x1c, e, h, x2c);
                    mo[u] = Msm[ptid + i * PNT];
                }
            }
#pragma unroll
            for (int u = 0; u < UB; u++) {
                const int i = i0 + u, idx = tid + i * NT;
                if (i < EPT && idx < ss) {
                    const float s_new = et * S[i] - th * g[u];
                    const float m_new = fmaf(keep, mo[u], s_new);
                    S[i] = s_new; Msm[ptid + i * PNT] = m_new;
                    sn[idx] = s_new;
                    if (!clamp) mn[idx] = m_new;
                    sq[0] = fmaf(m_new, m_new, sq[0]);
                }
            }
        }
        if (clamp) {      // Frobenius projection over the whole packed state (titans_lmm.rs:812-821)
            block_sum<1>(sq, red);
            const float norm = sqrtf(sq[0]);
            const float scale = norm > a.m_norm_max ? a.m_norm_max / norm : 1.0f;
#pragma unroll
            for (int i = 0; i < EPT; i++) {
                const int idx = tid + i * NT;
                if (idx < ss) { const float m = Msm[ptid + i * PNT] * scale; Msm[ptid + i * PNT] = m; mn[idx] = m; }
            }
        }
        __syncthreads();
        // y_t = MLP(M_{t+1}, q_t)
        rowdot(Msm, 0, dh, d, D.tps_d, qb, [&](int r, float s) { pre[P(r)] = act_fn<ACT>(s + Msm[P(D.o1 + r)]); });
        __syncthreads();
        rowdot(Msm, D.o2, d, dh, D.tps_h, pre, [&](int r, float s) { y[(size_t)t * d + r] = s + Msm[P(D.o3 + r)]; });
        // no barrier here: the next token stages kb | vb | qb, which nothing above still reads,
        // and its first barrier comes before pre or M are written again
    }
}

struct BwdArgs {
    const float *k, *v, *q, *alpha, *theta, *eta, *m_states, *s_states, *d_y;
    float *d_k, *d_v, *d_q, *d_alpha, *d_theta, *d_eta, *d_m_init, *d_s_init;
    int seq_len;
    long long in_stride, m_stride;
    Dims D;
};

inline int stage_floats(const Dims& D) { return D.o2 > D.ss - D.o2 ? D.o2 : D.ss - D.o2; }
inline size_t bwd_smem_floats(const Dims& D)
{
    return (size_t)padded(D.ss) + padded(stage_floats(D)) + 7 * padded(D.d) + 8 * padded(D.dh) + NT + 4 * NW;
}

// Reverse loop (titans_lmm.rs:896-1131). Per token, with dM, dS the gradients of M_{t+1}, S_{t+1}:
//   1 readout      pq = W1' q + b1', hq = act(pq); dpq = (W2'^T dy) act'(pq); d_q = W1'^T dpq
//                  dM += {dpq q^T, dpq, dy hq^T, dy}
//   2-4            dS += dM; d_alpha = -<M_t, dM>; d_eta = <S_t, dS>; d_theta = -<grad_t, dS>
//   5 (G = -theta dS)  adj = (G_W1 k + G_b1) act'(pre);  d_err = W2 adj + G_W2 h + G_b2
//                  inj1 = G_W2^T e;  inj0 = G_W1^T gp
//   6              d_v = -d_err;  d_pre = (W2^T d_err + inj1) act'(pre);  d_k = W1^T d_pre + inj0
//                  dM <- (1-alpha) dM + {d_pre k^T, d_pre, d_err h^T + e adj^T, d_err};  dS <- eta dS
// The activation's second derivative does not appear, as in the reference.
// Row products need their matrix in (padded) shared memory: {W1', b1'}, {W1, b1} and {W2, b2} pass
// through one staging buffer in turn; column sums read global memory directly (coalesced).
template <int ACT, int EPT, int SD, int SDH>
__global__ void __launch_bounds__(NT, 1) mlp_bwd_kernel(BwdArgs a)
{
    extern __shared__ __align__(16) float sm[];
    const Dims& D = a.D;
    const int d = SD ? SD : D.d, dh = SD ? SDH : D.dh, ss = SD ? 2 * SD * SDH + SD + SDH : D.ss;
    const int tid = threadIdx.x, b = blockIdx.x, ptid = P(tid);
    __builtin_assume(tid >= 0 && tid < NT);
    const int pd = padded(d), ph = padded(dh);
    float* dS = sm;                                   // padded packed state
    float* stg = dS + padded(ss);                     // staging: {W1, b1} or {W2, b2} of one state
    float* kb = stg + padded(D.o2 > ss - D.o2 ? D.o2 : ss - D.o2);
    float* vb = kb + pd;
    float* qb = vb + pd;
    float* dyb = qb + pd;
    float* e = dyb + pd;
    float* derr = e + pd;
    float* inj0 = derr + pd;
    float* pre = inj0 + pd;               // act'(pre)
    float* h = pre + ph;
    float* gp = h + ph;
    float* hq = gp + ph;
    float* dpq = hq + ph;                 // act'(pq), then dpq
    float* adj = dpq + ph;
    float* inj1 = adj + ph;
    float* dpre = inj1 + ph;
    float* scr = dpre + ph;
    float* red = scr + NT;

    const float* k = a.k + (size_t)b * a.in_stride;
    const float* v = a.v + (size_t)b * a.in_stride;
    const float* q = a.q + (size_t)b * a.in_stride;
    const float* dy = a.d_y + (size_t)b * a.in_stride;
    float* d_k = a.d_k + (size_t)b * a.in_stride;
    float* d_v = a.d_v + (size_t)b * a.in_stride;
    float* d_q = a.d_q + (size_t)b * a.in_stride;
    const size_t g0 = (size_t)b * a.seq_len;
    const float* mt = a.m_states + (size_t)b * a.m_stride;
    const float* st = a.s_states + (size_t)b * a.m_stride;
    const int gh_ = fd_div(tid, D.div_h), jh = tid - gh_ * dh, Gh = NT / dh;   // column split, C = dh
    const int gd_ = fd_div(tid, D.div_d), jd = tid - gd_ * d, Gd = NT / d;     // column split, C = d
    const int w2sz = d * dh;

    float dM[EPT];
#pragma unroll
    for (int i = 0; i < EPT; i++) {
        dM[i] = 0.0f;
        const int idx = tid + i * NT;
        if (idx < ss) dS[ptid + i * PNT] = 0.0f;
    }
    for (int t = a.seq_len - 1; t >= 0; t--) {
        const float* Mt = mt + (size_t)t * ss;
        const float* Mn = Mt + ss;
        const float* St = st + (size_t)t * ss;
        if (t > 0) {      // the states token t - 1 reads first (M_{t-1}, S_{t-1}) on their way into L2
            for (int f = tid * 32; f < ss; f += NT * 32) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(Mt - ss + f));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(St - ss + f));
            }
        }
        for (int i = tid; i < 4 * d; i += NT) {
            const int w = fd_div(i, D.div_d), c = i - w * d;
            (w == 0 ? kb : w == 1 ? vb : w == 2 ? qb : dyb)[P(c)] = (w == 0 ? k : w == 1 ? v : w == 2 ? q : dy)[(size_t)t * d + c];
        }
        const float al = a.alpha[g0 + t], th = a.theta[g0 + t], et = a.eta[g0 + t];
        // 1: readout through M_{t+1}
        stage(stg, Mn, D.o2);
        __syncthreads();
        rowdot(stg, 0, dh, d, D.tps_d, qb, [&](int r, float s) { const float p = s + stg[P(D.o1 + r)]; hq[P(r)] = act_fn<ACT>(p); dpq[P(r)] = act_prime<ACT>(p); });
        colsum<false>(Mn, D.o2, d, dh, dyb, scr, gh_, jh, Gh, [&](int j, float s) { dpq[P(j)] *= s; });
        colsum<true>(stg, 0, dh, d, dpq, scr, gd_, jd, Gd, [&](int j, float s) { d_q[(size_t)t * d + j] = s; });
        // 3: the inner gradient's vectors through M_t
        stage(stg, Mt, D.o2);
        __syncthreads();
        rowdot(stg, 0, dh, d, D.tps_d, kb, [&](int r, float s) { const float p = s + stg[P(D.o1 + r)]; h[P(r)] = act_fn<ACT>(p); pre[P(r)] = act_prime<ACT>(p); });
        __syncthreads();
        stage(stg, Mt + D.o2, ss - D.o2);
        __syncthreads();
        rowdot(stg, 0, d, dh, D.tps_h, h, [&](int r, float s) { e[P(r)] = s + stg[P(w2sz + r)] - vb[P(r)]; });
        __syncthreads();
        colsum<true>(stg, 0, d, dh, e, scr, gh_, jh, Gh, [&](int j, float s) { gp[P(j)] = s * pre[P(j)]; });
        // dM += readout terms; dS += dM; the three gate gradients
        float acc[3] = {0.0f, 0.0f, 0.0f};
        const int c1 = tid % (SD ? SD : 1), c2 = tid % (SDH ? SDH : 1);
        {
            const float q1c = SD ? qb[P(c1)] : 0.0f, hq2c = SD ? hq[P(c2)] : 0.0f;
            const float k1c = SD ? kb[P(c1)] : 0.0f, h2c = SD ? h[P(c2)] : 0.0f;
#pragma unroll
            for (int i0 = 0; i0 < EPT; i0 += UB) {
                float mv[UB], sv[UB], ro[UB], gr[UB], ds0[UB];
#pragma unroll
                for (int u = 0; u < UB; u++) {
                    const int i = i0 + u, idx = tid + i * NT;
                    if (i < EPT && idx < ss) {
                        mv[u] = Mt[idx]; sv[u] = St[idx];
                        ro[u] = outer_term<SD, SDH>(D, idx, dpq, qb, q1c, dyb, hq, hq2c);
                        gr[u] = outer_term<SD, SDH>(D, idx, gp, kb, k1c, e, h, h2c);
                        ds0[u] = dS[ptid + i * PNT];
                    }
                }
#pragma unroll
                for (int u = 0; u < UB; u++) {
                    const int i = i0 + u, idx = tid + i * NT;
                    if (i < EPT && idx < ss) {
                        const float dm = dM[i] + ro[u];
                        const float ds = ds0[u] + dm;
                        dM[i] = dm; dS[ptid + i * PNT] = ds;
                        acc[0] = fmaf(mv[u], dm, acc[0]);
                        acc[1] = fmaf(sv[u], ds, acc[1]);
                        acc[2] = fmaf(gr[u], ds, acc[2]);
                    }
                }
            }
        }
        block_sum<3>(acc, red);          // its barriers also publish dS
        if (tid == 0) { a.d_alpha[g0 + t] = -acc[0]; a.d_eta[g0 + t] = acc[1]; a.d_theta[g0 + t] = -acc[2]; }
        // 5: products with G = -theta dS
        rowdot(dS, 0, dh, d, D.tps_d, kb, [&](int r, float s) { adj[P(r)] = -th * (s + dS[P(D.o1 + r)]) * pre[P(r)]; });
        rowdot(dS, D.o2, d, dh, D.tps_h, h, [&](int r, float s) { derr[P(r)] = -th * (s + dS[P(D.o3 + r)]); });
        colsum<true>(dS, D.o2, d, dh, e, scr, gh_, jh, Gh, [&](int j, float s) { inj1[P(j)] = -th * s; });
        // (the barriers of colsum published adj and derr)
        rowdot(stg, 0, d, dh, D.tps_h, adj, [&](int r, float s) { derr[P(r)] += s; });
        __syncthreads();
        if (tid < d) d_v[(size_t)t * d + tid] = -derr[P(tid)];
        colsum<true>(stg, 0, d, dh, derr, scr, gh_, jh, Gh, [&](int j, float s) { dpre[P(j)] = (s + inj1[P(j)]) * pre[P(j)]; });
        colsum<true>(dS, 0, dh, d, gp, scr, gd_, jd, Gd, [&](int j, float s) { inj0[P(j)] = -th * s; });
        colsum<false>(Mt, 0, dh, d, dpre, scr, gd_, jd, Gd, [&](int j, float s) { d_k[(size_t)t * d + j] = s + inj0[P(j)]; });
        // 6: carry to token t - 1
        const float keep = 1.0f - al;
        {
            const float k1c = SD ? kb[P(c1)] : 0.0f, h2c = SD ? h[P(c2)] : 0.0f, adj2c = SD ? adj[P(c2)] : 0.0f;
            const int o2 = SD ? SDH * SD + SDH : D.o2, o3 = o2 + d * dh;
#pragma unroll
            for (int i0 = 0; i0 < EPT; i0 += UB) {
                float add[UB], ds0[UB];
#pragma unroll
                for (int u = 0; u < UB; u++) {
                    const int i = i0 + u, idx = tid + i * NT;
                    if (i < EPT && idx < ss) {
                        add[u] = outer_term<SD, SDH>(D, idx, dpre, kb, k1c, derr, h, h2c);
                        if (idx >= o2 && idx < o3) {          // cross term e adj^T of W2
                            const int el = idx - o2, r = SD ? el / (SDH ? SDH : 1) : fd_div(el, D.div_h);
                            add[u] = fmaf(e[P(r)], SD ? adj2c : adj[P(el - r * dh)], add[u]);
                        }
                        ds0[u] = dS[ptid + i * PNT];
                    }
                }
#pragma unroll
                for (int u = 0; u < UB; u++) {
                    const int i = i0 + u, idx = tid + i * NT;
                    if (i < EPT && idx < ss) {
                        dM[i] = fmaf(keep, dM[i], add[u]);
                        dS[ptid + i * PNT] = ds0[u] * et;
                    }
                }
            }
        }
        __syncthreads();
    }
    // summed over the batch, like the reference (titans_mlp_backward.cu:557-561); caller pre-zeroes
#pragma unroll
    for (int i = 0; i < EPT; i++) {
        const int idx = tid + i * NT;
        if (idx < ss) {
            atomicAdd(a.d_m_init + idx, dM[i]);
            atomicAdd(a.d_s_init + idx, dS[ptid + i * PNT]);
        }
    }
}

// ───────────────────── static head size: d = 64, d_hidden = 256 ─────────────────────
// The reference's head size with its default expansion factor 4. Everything is float4: the packed
// state is 8272 float4 (17 per thread), region borders fall on float4 borders, and for the float4
// q = tid + 512 i of one thread the columns are fixed (W1: 4 (tid % 16), W2: 4 (tid % 64)), so the
// vector operand of every outer product sits in four registers for a whole pass and only the row
// scalar is read per element. Shared memory is unpadded; row products read 16-byte chunks in an
// order rotated by the lane, which spreads a quarter-warp over all eight 16-byte bank groups.
namespace s64 {
constexpr int D = 64, DH = 256, O1 = DH * D, O2 = O1 + DH, O3 = O2 + D * DH, SS = O3 + D;
constexpr int NV = SS / 4, V = (NV + NT - 1) / NT;                 // 8272 float4, 17 per thread
constexpr int SCR = 2048;
#ifndef NLH_MLP_PB
#define NLH_MLP_PB 2
#endif
constexpr int PB = NLH_MLP_PB;      // float4 per thread whose loads are issued together in the backward's first pass

__device__ __forceinline__ float4 f4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 mul4(float s, float4 a) { return make_float4(s * a.x, s * a.y, s * a.z, s * a.w); }
__device__ __forceinline__ float4 fma4(float s, float4 a, float4 b) { return make_float4(fmaf(s, a.x, b.x), fmaf(s, a.y, b.y), fmaf(s, a.z, b.z), fmaf(s, a.w, b.w)); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float dot4(float4 a, float4 b, float acc) { return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, fmaf(a.w, b.w, acc)))); }
__device__ __forceinline__ bool live(int i, int tid) { return i < V - 1 || tid < NV - (V - 1) * NT; }

// Outer-product term of float4 number tid + NT * i of the packed state (i is a compile-time
// constant after unrolling): W1 -> a1[row] x1v, b1 -> a1, W2 -> a2[row] x2v, b2 -> a2.
__device__ __forceinline__ float4 term4(int i, int tid, const float* a1, float4 x1v, const float* a2, float4 x2v)
{
    if (i < 8) return mul4(a1[(tid >> 4) + 32 * i], x1v);
    if (i == 8 && tid < 64) return f4(a1 + 4 * tid);
    if (i == V - 1 && tid >= 64) return f4(a2 + 4 * (tid - 64));
    return mul4(a2[((tid - 64) >> 6) + 8 * (i - 8)], x2v);
}
__device__ __forceinline__ bool in_w2(int i, int tid) { return (i == 8 && tid >= 64) || (i > 8 && i < V - 1) || (i == V - 1 && tid < 64); }

// out(r) = sum_c W[r, c] x[c]; W [R, C] in shared memory, 2^tps threads per row (C = 32 << tps,
// R << tps = NT). epi(r, sum) on the first thread of each row.
template <class Epi>
__device__ __forceinline__ void rowdot(const float* W, int C, int tps, const float* x, Epi epi)
{
    const int tid = threadIdx.x, r = tid >> tps, p = tid & ((1 << tps) - 1), lane = tid & 31;
    const float* w = W + r * C + 32 * p;
    const float* xs = x + 32 * p;
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int jj = 0; jj < 8; jj += 2) {
        const int c0 = 4 * ((jj + lane) & 7), c1 = 4 * ((jj + 1 + lane) & 7);
        a0 = dot4(f4(w + c0), f4(xs + c0), a0);
        a1 = dot4(f4(w + c1), f4(xs + c1), a1);
    }
    float acc = a0 + a1;
    for (int o = (1 << tps) >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (p == 0) epi(r, acc);
}

// Two products with the same matrix in one pass over it: s0 = W x0, s1 = W x1.
template <class Epi>
__device__ __forceinline__ void rowdot2(const float* W, int C, int tps, const float* x0, const float* x1, Epi epi)
{
    const int tid = threadIdx.x, r = tid >> tps, p = tid & ((1 << tps) - 1), lane = tid & 31;
    const float* w = W + r * C + 32 * p;
    const float* xa = x0 + 32 * p;
    const float* xb = x1 + 32 * p;
    float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll
    for (int jj = 0; jj < 8; jj += 2) {
        const int c0 = 4 * ((jj + lane) & 7), c1 = 4 * ((jj + 1 + lane) & 7);
        const float4 w0 = f4(w + c0), w1 = f4(w + c1);
        a0 = dot4(w0, f4(xa + c0), a0); b0 = dot4(w0, f4(xb + c0), b0);
        a1 = dot4(w1, f4(xa + c1), a1); b1 = dot4(w1, f4(xb + c1), b1);
    }
    float sa = a0 + a1, sb = b0 + b1;
    for (int o = (1 << tps) >> 1; o > 0; o >>= 1) {
        sa += __shfl_xor_sync(0xffffffffu, sa, o);
        sb += __shfl_xor_sync(0xffffffffu, sb, o);
    }
    if (p == 0) epi(r, sa, sb);
}

// out(j) = sum_i W[i, j] x[i]; W [R, C] in shared or global memory (16-byte aligned rows), x in
// shared memory. Thread (g, cg): 8 consecutive rows, 4 consecutive columns; the NT / (C / 4) partial
// float4 sums meet in scr[SCR]; epi(j, sum) on threads j < C. Two block barriers inside.
template <class Epi>
__device__ __forceinline__ void colsum(const float* __restrict__ W, int C, int lgcg, const float* x, float* scr, Epi epi)
{
    const int tid = threadIdx.x, cg = tid & ((1 << lgcg) - 1), g = tid >> lgcg;
    const float* w = W + (size_t)(8 * g) * C + 4 * cg;
    const float4 xa = f4(x + 8 * g), xb = f4(x + 8 * g + 4);
    float4 wv[4];
#pragma unroll
    for (int u = 0; u < 4; u++) wv[u] = f4(w + (size_t)u * C);
    float4 acc = mul4(xa.x, wv[0]);
    acc = fma4(xa.y, wv[1], acc); acc = fma4(xa.z, wv[2], acc); acc = fma4(xa.w, wv[3], acc);
#pragma unroll
    for (int u = 0; u < 4; u++) wv[u] = f4(w + (size_t)(u + 4) * C);
    acc = fma4(xb.x, wv[0], acc); acc = fma4(xb.y, wv[1], acc); acc = fma4(xb.z, wv[2], acc); acc = fma4(xb.w, wv[3], acc);
    *reinterpret_cast<float4*>(scr + g * C + 4 * cg) = acc;
    __syncthreads();
    if (tid < C) {
        const int G = NT >> lgcg;
        float s0 = 0.0f, s1 = 0.0f;
        for (int gg = 0; gg < G; gg += 2) { s0 += scr[gg * C + tid]; s1 += scr[(gg + 1) * C + tid]; }
        epi(tid, s0 + s1);
    }
    __syncthreads();
}

// nv float4 of global memory into shared memory
__device__ __forceinline__ void stage(float* dst, const float* __restrict__ src, int nv)
{
    const int tid = threadIdx.x;
#pragma unroll
    for (int u0 = 0; u0 < 9; u0 += 3) {
        float4 v[3];
#pragma unroll
        for (int u = 0; u < 3; u++) if (tid + (u0 + u) * NT < nv) v[u] = f4(src + 4 * (tid + (u0 + u) * NT));
#pragma unroll
        for (int u = 0; u < 3; u++) if (tid + (u0 + u) * NT < nv) *reinterpret_cast<float4*>(dst + 4 * (tid + (u0 + u) * NT)) = v[u];
    }
}

// Two column sums with the same matrix in one pass: s0 = W^T x0, s1 = W^T x1. scr: 2 * SCR floats.
template <class Epi>
__device__ __forceinline__ void colsum2(const float* __restrict__ W, int C, int lgcg, const float* x0, const float* x1,
                                        float* scr, Epi epi)
{
    const int tid = threadIdx.x, cg = tid & ((1 << lgcg) - 1), g = tid >> lgcg;
    const float* w = W + (size_t)(8 * g) * C + 4 * cg;
    float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        float4 wv[4];
#pragma unroll
        for (int u = 0; u < 4; u++) wv[u] = f4(w + (size_t)(4 * half + u) * C);
        const float4 xa = f4(x0 + 8 * g + 4 * half), xb = f4(x1 + 8 * g + 4 * half);
        acc0 = fma4(xa.x, wv[0], acc0); acc0 = fma4(xa.y, wv[1], acc0); acc0 = fma4(xa.z, wv[2], acc0); acc0 = fma4(xa.w, wv[3], acc0);
        acc1 = fma4(xb.x, wv[0], acc1); acc1 = fma4(xb.y, wv[1], acc1); acc1 = fma4(xb.z, wv[2], acc1); acc1 = fma4(xb.w, wv[3], acc1);
    }
    *reinterpret_cast<float4*>(scr + g * C + 4 * cg) = acc0;
    *reinterpret_cast<float4*>(scr + SCR + g * C + 4 * cg) = acc1;
    __syncthreads();
    if (tid < C) {
        const int G = NT >> lgcg;
        float s0 = 0.0f, s1 = 0.0f;
        for (int gg = 0; gg < G; gg++) { s0 += scr[gg * C + tid]; s1 += scr[SCR + gg * C + tid]; }
        epi(tid, s0, s1);
    }
    __syncthreads();
}

// nv float4 of global memory into shared memory with 16-byte asynchronous copies, all in flight at
// once; the caller's barrier after it makes them visible.
__device__ __forceinline__ void stage_async(float* dst, const float* __restrict__ src, int nv)
{
    const int tid = threadIdx.x;
#pragma unroll
    for (int u = 0; u < 9; u++) {
        const int qi = tid + u * NT;
        if (qi < nv) {
            const unsigned d32 = (unsigned)__cvta_generic_to_shared(dst + 4 * qi);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d32), "l"(src + 4 * qi) : "memory");
        }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}
__device__ __forceinline__ void stage_wait() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

inline size_t fwd_smem_floats() { return (size_t)SS + 7 * D + 4 * DH + SCR + 4 * NW; }
inline size_t bwd_smem_floats() { return (size_t)SS + O2 + 11 * D + 10 * DH + 2 * SCR + 4 * NW; }

// Token loop, rotated: M_{t+1} serves the readout of token t AND the prediction of token t + 1, so
// both row products with W1' (on q_t and k_{t+1}) share one pass over the matrix, and both with W2'
// (on act(W1' q_t + b1') and h_{t+1}) the next. A token is then four phases: column sum, update,
// two double row products. k, v, q of token t + 1 are fetched at the top of token t.
template <int ACT>
__global__ void __launch_bounds__(NT, 1) mlp_fwd64_kernel(FwdArgs a)
{
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, b = blockIdx.x;
    float* Msm = sm;
    float* kvq = Msm + SS;                // two buffers of k | v | q (token parity)
    float* e = kvq + 6 * D;
    float* pre = e + D;
    float* h = pre + DH;
    float* gp = h + DH;
    float* hq = gp + DH;
    float* scr = hq + DH;
    float* red = scr + SCR;
    const float* k = a.k + (size_t)b * a.in_stride;
    const float* v = a.v + (size_t)b * a.in_stride;
    const float* q = a.q + (size_t)b * a.in_stride;
    float* y = a.y + (size_t)b * a.in_stride;
    const float* alpha = a.alpha + (size_t)b * a.seq_len;
    const float* theta = a.theta + (size_t)b * a.seq_len;
    const float* eta = a.eta + (size_t)b * a.seq_len;
    float* mt = a.m_states + (size_t)b * a.m_stride;
    float* st = a.s_states + (size_t)b * a.m_stride;
    const bool clamp = m_norm_enabled(a.m_norm_max);
    float4* M4 = reinterpret_cast<float4*>(Msm);
    const float* src = tid < D ? k : tid < 2 * D ? v : q;     // stream this thread stages (tid < 3 D)

    float4 S4[V];
#pragma unroll
    for (int i = 0; i < V; i++) {
        S4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live(i, tid)) {
            const int qi = tid + i * NT;
            const float4 m = f4(a.m_init + (size_t)b * SS + 4 * qi);
            S4[i] = f4(a.s_init + (size_t)b * SS + 4 * qi);
            M4[qi] = m;
            reinterpret_cast<float4*>(mt)[qi] = m;
            reinterpret_cast<float4*>(st)[qi] = S4[i];
        }
    }
    if (a.seq_len == 0) return;
    if (tid < 3 * D) kvq[tid] = src[tid & (D - 1)];
    __syncthreads();
    rowdot(Msm, D, 1, kvq, [&](int r, float s) { const float p = s + Msm[O1 + r]; pre[r] = p; h[r] = act_fn<ACT>(p); });
    __syncthreads();
    rowdot(Msm + O2, DH, 3, h, [&](int r, float s) { e[r] = s + Msm[O3 + r] - kvq[D + r]; });
    __syncthreads();
    for (int t = 0; t < a.seq_len; t++) {
        float* cur = kvq + (t & 1) * 3 * D;
        float* nxt = kvq + ((t + 1) & 1) * 3 * D;
        const bool has_next = t + 1 < a.seq_len;
        float staged = 0.0f;
        if (has_next && tid < 3 * D) staged = src[(size_t)(t + 1) * D + (tid & (D - 1))];
        const float al = alpha[t], th = theta[t], et = eta[t];
        colsum(Msm + O2, DH, 6, e, scr, [&](int j, float s) { gp[j] = s * act_prime<ACT>(pre[j]); });
        float4* mn = reinterpret_cast<float4*>(mt + (size_t)(t + 1) * SS);
        float4* sn = reinterpret_cast<float4*>(st + (size_t)(t + 1) * SS);
        float sq[1] = {0.0f};
        const float keep = 1.0f - al;
        const float4 x1v = f4(cur + 4 * (tid & 15)), x2v = f4(h + 4 * (tid & 63));
#pragma unroll
        for (int i0 = 0; i0 < V; i0 += 4) {
            float4 g[4], mo[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u;
                if (i < V && live(i, tid)) { g[u] = term4(i, tid, gp, x1v, e, x2v); mo[u] = M4[tid + i * NT]; }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u;
                if (i < V && live(i, tid)) {
                    const float4 s_new = fma4(-th, g[u], mul4(et, S4[i]));
                    const float4 m_new = fma4(keep, mo[u], s_new);
                    S4[i] = s_new; M4[tid + i * NT] = m_new;
                    sn[tid + i * NT] = s_new;
                    if (!clamp) mn[tid + i * NT] = m_new;
                    sq[0] = dot4(m_new, m_new, sq[0]);
                }
            }
        }
        if (clamp) {      // Frobenius projection over the whole packed state (titans_lmm.rs:812-821)
            block_sum<1>(sq, red);
            const float norm = sqrtf(sq[0]);
            const float scale = norm > a.m_norm_max ? a.m_norm_max / norm : 1.0f;
#pragma unroll
            for (int i = 0; i < V; i++)
                if (live(i, tid)) { const float4 m = mul4(scale, M4[tid + i * NT]); M4[tid + i * NT] = m; mn[tid + i * NT] = m; }
        }
        if (tid < 3 * D) nxt[tid] = staged;
        __syncthreads();
        // W1': readout hidden of q_t, prediction hidden of k_{t+1}
        rowdot2(Msm, D, 1, cur + 2 * D, nxt, [&](int r, float sq_, float sk) {
            const float b1 = Msm[O1 + r];
            hq[r] = act_fn<ACT>(sq_ + b1);
            if (has_next) { const float p = sk + b1; pre[r] = p; h[r] = act_fn<ACT>(p); }
        });
        __syncthreads();
        // W2': y_t and the error of token t + 1
        rowdot2(Msm + O2, DH, 3, hq, h, [&](int r, float sy, float se) {
            const float b2 = Msm[O3 + r];
            y[(size_t)t * D + r] = sy + b2;
            if (has_next) e[r] = se + b2 - nxt[D + r];
        });
        __syncthreads();
    }
}

// Reverse loop, rotated like the forward: M_t serves the inner gradient of token t AND the readout
// of token t - 1 (whose M_{t+1} it is). Iteration t stages {W1_t, b1_t} once for the row products on
// k_t and q_{t-1}, then {W2_t, b2_t} for e_t, the column sums on e_t and dy_{t-1}, and phase 5; the
// readout vectors of token t - 1 wait in the other half of a double buffer for iteration t - 1.
template <int ACT>
__global__ void __launch_bounds__(NT, 1) mlp_bwd64_kernel(BwdArgs a)
{
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, b = blockIdx.x;
    float* dS = sm;
    float* stg = dS + SS;                 // {W1, b1} (O2 floats) or {W2, b2} of one state
    float* vec = stg + O2;                // two buffers of k | v | q | dy (token parity)
    float* e = vec + 8 * D;
    float* derr = e + D;
    float* inj0 = derr + D;
    float* pre = inj0 + D;                // act'(pre)
    float* h = pre + DH;
    float* gp = h + DH;
    float* hqb = gp + DH;                 // two buffers (token parity)
    float* dpqb = hqb + 2 * DH;           // two buffers: act'(pq), then dpq
    float* adj = dpqb + 2 * DH;
    float* inj1 = adj + DH;
    float* dpre = inj1 + DH;
    float* scr = dpre + DH;               // 2 * SCR
    float* red = scr + 2 * SCR;
    const float* k = a.k + (size_t)b * a.in_stride;
    const float* v = a.v + (size_t)b * a.in_stride;
    const float* q = a.q + (size_t)b * a.in_stride;
    const float* dy = a.d_y + (size_t)b * a.in_stride;
    float* d_k = a.d_k + (size_t)b * a.in_stride;
    float* d_v = a.d_v + (size_t)b * a.in_stride;
    float* d_q = a.d_q + (size_t)b * a.in_stride;
    const size_t g0 = (size_t)b * a.seq_len;
    const float* mt = a.m_states + (size_t)b * a.m_stride;
    const float* st = a.s_states + (size_t)b * a.m_stride;
    float4* dS4 = reinterpret_cast<float4*>(dS);
    const float* src = tid < D ? k : tid < 2 * D ? v : tid < 3 * D ? q : dy;    // stream staged by this thread (tid < 4 D)
    const int S = a.seq_len;

    float4 dM4[V];
#pragma unroll
    for (int i = 0; i < V; i++) {
        dM4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live(i, tid)) dS4[tid + i * NT] = dM4[i];
    }
    // dS of the next token is eta_t x (dS of this one): the factor is applied when the next token
    // reads dS in its element pass, so the carry step never touches the shared copy
    float ds_scale = 1.0f;
    if (S > 0) {      // readout of the last token through the final state M_S
        const int cur = (S - 1) & 1;
        const float* Mn = mt + (size_t)S * SS;
        float* vc = vec + cur * 4 * D;
        if (tid < 4 * D) vc[tid] = src[(size_t)(S - 1) * D + (tid & (D - 1))];
        stage_async(stg, Mn, O2 / 4);
        stage_wait();
        __syncthreads();
        float* hq = hqb + cur * DH;
        float* dpq = dpqb + cur * DH;
        rowdot(stg, D, 1, vc + 2 * D, [&](int r, float s) { const float p = s + stg[O1 + r]; hq[r] = act_fn<ACT>(p); dpq[r] = act_prime<ACT>(p); });
        colsum(Mn + O2, DH, 6, vc + 3 * D, scr, [&](int j, float s) { dpq[j] *= s; });
        colsum(stg, D, 4, dpq, scr, [&](int j, float s) { d_q[(size_t)(S - 1) * D + j] = s; });
    }
    for (int t = S - 1; t >= 0; t--) {
        const float* Mt = mt + (size_t)t * SS;
        const float* St = st + (size_t)t * SS;
        const int cur = t & 1, prv = cur ^ 1;
        const bool has_prev = t > 0;
        float* vc = vec + cur * 4 * D;        // k_t | v_t | q_t | dy_t
        float* vp = vec + prv * 4 * D;        // the same of token t - 1
        float* hq = hqb + cur * DH;
        float* dpq = dpqb + cur * DH;
        float* hq_p = hqb + prv * DH;
        float* dpq_p = dpqb + prv * DH;
        float staged = 0.0f;
        if (has_prev && tid < 4 * D) staged = src[(size_t)(t - 1) * D + (tid & (D - 1))];
        const float al = a.alpha[g0 + t], th = a.theta[g0 + t], et = a.eta[g0 + t];
        stage_async(stg, Mt, O2 / 4);
        if (has_prev) {
            // what token t - 1 reads first (M_{t-1}, S_{t-1}; the streams of token t - 2) on its way into L2
            for (int f = tid * 32; f < SS; f += NT * 32) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(Mt - SS + f));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(St - SS + f));
            }
            if (t > 1 && tid < 4 * D && (tid & 31) == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + (size_t)(t - 2) * D + (tid & (D - 1))));
            if (tid < 4 * D) vp[tid] = staged;
        }
        stage_wait();
        __syncthreads();
        // W1_t: hidden of k_t (inner gradient of token t) and of q_{t-1} (readout of token t - 1)
        rowdot2(stg, D, 1, vc, vp + 2 * D, [&](int r, float sk, float sq_) {
            const float b1 = stg[O1 + r];
            const float p = sk + b1;
            h[r] = act_fn<ACT>(p); pre[r] = act_prime<ACT>(p);
            if (has_prev) { const float pq = sq_ + b1; hq_p[r] = act_fn<ACT>(pq); dpq_p[r] = act_prime<ACT>(pq); }
        });
        __syncthreads();
        stage_async(stg, Mt + O2, (SS - O2) / 4);
        stage_wait();
        __syncthreads();
        rowdot(stg, DH, 3, h, [&](int r, float s) { e[r] = s + stg[D * DH + r] - vc[D + r]; });
        __syncthreads();
        // W2_t^T on e_t (-> gp) and on dy_{t-1} (-> dpq of token t - 1)
        colsum2(stg, DH, 6, e, vp + 3 * D, scr, [&](int j, float s0, float s1) {
            gp[j] = s0 * pre[j];
            if (has_prev) dpq_p[j] *= s1;
        });
        // dM += readout terms of token t; dS += dM; the three gate gradients
        float acc[3] = {0.0f, 0.0f, 0.0f};
        {
            const float4 q1v = f4(vc + 2 * D + 4 * (tid & 15)), hq2v = f4(hq + 4 * (tid & 63));
            const float4 k1v = f4(vc + 4 * (tid & 15)), h2v = f4(h + 4 * (tid & 63));
            const float4* Mt4 = reinterpret_cast<const float4*>(Mt);
            const float4* St4 = reinterpret_cast<const float4*>(St);
            const float4* stg4 = reinterpret_cast<const float4*>(stg);
#pragma unroll
            for (int i0 = 0; i0 < V; i0 += PB) {
                float4 mv[PB], sv[PB], ro[PB], gr[PB], ds0[PB];
#pragma unroll
                for (int u = 0; u < PB; u++) {
                    const int i = i0 + u;
                    if (i < V && live(i, tid)) {
                        // the {W2, b2} half of M_t is in the staging buffer at this point
                        const bool staged_half = i > 8 || (i == 8 && tid >= 64);
                        mv[u] = staged_half ? stg4[tid + i * NT - O2 / 4] : Mt4[tid + i * NT];
                        sv[u] = St4[tid + i * NT];
                        ro[u] = term4(i, tid, dpq, q1v, vc + 3 * D, hq2v);
                        gr[u] = term4(i, tid, gp, k1v, e, h2v);
                        ds0[u] = dS4[tid + i * NT];
                    }
                }
#pragma unroll
                for (int u = 0; u < PB; u++) {
                    const int i = i0 + u;
                    if (i < V && live(i, tid)) {
                        const float4 dm = add4(dM4[i], ro[u]);
                        const float4 ds = fma4(ds_scale, ds0[u], dm);
                        dM4[i] = dm; dS4[tid + i * NT] = ds;
                        acc[0] = dot4(mv[u], dm, acc[0]);
                        acc[1] = dot4(sv[u], ds, acc[1]);
                        acc[2] = dot4(gr[u], ds, acc[2]);
                    }
                }
            }
        }
        block_sum<3>(acc, red);          // its barriers also publish dS
        if (tid == 0) { a.d_alpha[g0 + t] = -acc[0]; a.d_eta[g0 + t] = acc[1]; a.d_theta[g0 + t] = -acc[2]; }
        // 5: products with G = -theta dS
        rowdot(dS, D, 1, vc, [&](int r, float s) { adj[r] = -th * (s + dS[O1 + r]) * pre[r]; });
        rowdot(dS + O2, DH, 3, h, [&](int r, float s) { derr[r] = -th * (s + dS[O3 + r]); });
        colsum(dS + O2, DH, 6, e, scr, [&](int j, float s) { inj1[j] = -th * s; });
        rowdot(stg, DH, 3, adj, [&](int r, float s) { derr[r] += s; });
        __syncthreads();
        if (tid < D) d_v[(size_t)t * D + tid] = -derr[tid];
        colsum(stg, DH, 6, derr, scr, [&](int j, float s) { dpre[j] = (s + inj1[j]) * pre[j]; });
        colsum(dS, D, 4, gp, scr, [&](int j, float s) { inj0[j] = -th * s; });
        // W1_t^T on d_pre (-> d_k of token t) and on dpq of token t - 1 (-> its d_q)
        colsum2(Mt, D, 4, dpre, dpq_p, scr, [&](int j, float s0, float s1) {
            d_k[(size_t)t * D + j] = s0 + inj0[j];
            if (has_prev) d_q[(size_t)(t - 1) * D + j] = s1;
        });
        // 6: carry to token t - 1
        const float keep = 1.0f - al;
        {
            const float4 k1v = f4(vc + 4 * (tid & 15)), h2v = f4(h + 4 * (tid & 63)), adjv = f4(adj + 4 * (tid & 63));
#pragma unroll
            for (int i = 0; i < V; i++) {
                if (live(i, tid)) {
                    float4 add = term4(i, tid, dpre, k1v, derr, h2v);
                    if (in_w2(i, tid)) add = fma4(e[((tid - 64) >> 6) + 8 * (i - 8)], adjv, add);   // cross term e adj^T
                    dM4[i] = fma4(keep, dM4[i], add);
                }
            }
        }
        ds_scale = et;
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < V; i++) {
        if (live(i, tid)) {
            const int f = 4 * (tid + i * NT);
            const float4 ds = mul4(ds_scale, dS4[tid + i * NT]);
            atomicAdd(a.d_m_init + f, dM4[i].x); atomicAdd(a.d_m_init + f + 1, dM4[i].y);
            atomicAdd(a.d_m_init + f + 2, dM4[i].z); atomicAdd(a.d_m_init + f + 3, dM4[i].w);
            atomicAdd(a.d_s_init + f, ds.x); atomicAdd(a.d_s_init + f + 1, ds.y);
            atomicAdd(a.d_s_init + f + 2, ds.z); atomicAdd(a.d_s_init + f + 3, ds.w);
        }
    }
}
}  // namespace s64

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

constexpr int EPT_SMALL = 17, EPT_LARGE = 65;     // packed-state elements per thread

static const char* unsupported(int d, int dh)
{
    if (d <= 0 || dh <= 0) return "d and d_hidden must be > 0";
    if (d > NT || dh > NT) return "d and d_hidden above 512 are not supported by the on-chip kernels";
    if ((long long)dh * d * 2 + dh + d > (long long)EPT_LARGE * NT ||
        bwd_smem_floats(make_dims(d, dh)) * sizeof(float) > 227 * 1024)
        return "packed MLP state above 33280 floats (d = 64, d_hidden = 256) does not fit on one SM";
    return nullptr;
}

template <int ACT>
static bool launch_fwd(const FwdArgs& a, int batch, cudaStream_t st)
{
    const size_t smem = fwd_smem_floats(a.D) * sizeof(float);
    if (a.D.d == 64 && a.D.dh == 256 && a.in_stride % 4 == 0 && a.m_stride % 4 == 0 && aligned16(a.m_init) &&
        aligned16(a.s_init) && aligned16(a.m_states) && aligned16(a.s_states)) {
        // the reference's head size and expansion: the float4 kernels
        const size_t sm64 = s64::fwd_smem_floats() * sizeof(float);
        cudaFuncSetAttribute(s64::mlp_fwd64_kernel<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm64);
        s64::mlp_fwd64_kernel<ACT><<<batch, NT, sm64, st>>>(a);
    } else if (a.D.ss <= EPT_SMALL * NT) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(mlp_fwd_kernel<ACT, EPT_SMALL, 0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mlp_fwd_kernel<ACT, EPT_SMALL, 0, 0><<<batch, NT, smem, st>>>(a);
    } else {
        cudaFuncSetAttribute(mlp_fwd_kernel<ACT, EPT_LARGE, 0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mlp_fwd_kernel<ACT, EPT_LARGE, 0, 0><<<batch, NT, smem, st>>>(a);
    }
    return check_launch("mlp_fwd_kernel");
}

template <int ACT>
static bool launch_bwd(const BwdArgs& a, int batch, cudaStream_t st)
{
    const size_t smem = bwd_smem_floats(a.D) * sizeof(float);
    if (a.D.d == 64 && a.D.dh == 256 && a.in_stride % 4 == 0 && a.m_stride % 4 == 0 && aligned16(a.m_states) &&
        aligned16(a.s_states)) {
        const size_t sm64 = s64::bwd_smem_floats() * sizeof(float);
        cudaFuncSetAttribute(s64::mlp_bwd64_kernel<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm64);
        s64::mlp_bwd64_kernel<ACT><<<batch, NT, sm64, st>>>(a);
    } else if (a.D.ss <= EPT_SMALL * NT) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(mlp_bwd_kernel<ACT, EPT_SMALL, 0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mlp_bwd_kernel<ACT, EPT_SMALL, 0, 0><<<batch, NT, smem, st>>>(a);
    } else {
        cudaFuncSetAttribute(mlp_bwd_kernel<ACT, EPT_LARGE, 0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mlp_bwd_kernel<ACT, EPT_LARGE, 0, 0><<<batch, NT, smem, st>>>(a);
    }
    return check_launch("mlp_bwd_kernel");
}

}  // namespace mlpm
}  // namespace nlh

using namespace nlh;

extern "C" {

void titans_mlp_forward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* eta, const float* m_initial, const float* s_initial, float* m_states,
    float* s_states, float* y, int32_t seq_len, int32_t d, int32_t d_hidden, int32_t batch_size,
    int32_t input_stride, int32_t m_stride, int32_t activation, float m_norm_max)
{
    const char* where = "titans_mlp_forward_f32_cuda";
    if (const char* why = mlpm::unsupported(d, d_hidden)) { record_status(d <= 0 || d_hidden <= 0 ? NLH_ERR_INVALID_ARG : NLH_ERR_UNSUPPORTED, where, why); return; }
    if (activation < 0 || activation > 2 || seq_len < 0 || batch_size < 0) { record_status(NLH_ERR_INVALID_ARG, where, "activation must be 0 (GELU), 1 (SiLU) or 2 (ReLU); seq_len, batch_size >= 0"); return; }
    if (batch_size == 0) return;
    mlpm::FwdArgs a{k_mem, v_mem, q_mem, alpha, theta, eta, m_initial, s_initial, m_states, s_states, y, seq_len,
                    (long long)input_stride, (long long)m_stride, m_norm_max, mlpm::make_dims(d, d_hidden)};
    cudaStream_t st = current_stream();
    if (activation == mlpm::ACT_GELU) mlpm::launch_fwd<mlpm::ACT_GELU>(a, batch_size, st);
    else if (activation == mlpm::ACT_SILU) mlpm::launch_fwd<mlpm::ACT_SILU>(a, batch_size, st);
    else mlpm::launch_fwd<mlpm::ACT_RELU>(a, batch_size, st);
}

void titans_mlp_backward_f32_cuda(const float* k_mem, const float* v_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* eta, const float* m_states, const float* s_states, const float* d_y,
    float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha, float* d_theta, float* d_eta,
    float* d_m_initial, float* d_s_initial, int32_t seq_len, int32_t d, int32_t d_hidden, int32_t batch_size,
    int32_t input_stride, int32_t m_stride, int32_t activation, float m_norm_max)
{
    (void)m_norm_max;   // gradients pass straight through the projection, as in the reference
    const char* where = "titans_mlp_backward_f32_cuda";
    if (const char* why = mlpm::unsupported(d, d_hidden)) { record_status(d <= 0 || d_hidden <= 0 ? NLH_ERR_INVALID_ARG : NLH_ERR_UNSUPPORTED, where, why); return; }
    if (activation < 0 || activation > 2 || seq_len < 0 || batch_size < 0) { record_status(NLH_ERR_INVALID_ARG, where, "activation must be 0 (GELU), 1 (SiLU) or 2 (ReLU); seq_len, batch_size >= 0"); return; }
    if (batch_size == 0) return;
    mlpm::BwdArgs a{k_mem, v_mem, q_mem, alpha, theta, eta, m_states, s_states, d_y, d_k_mem, d_v_mem, d_q_mem,
                    d_alpha, d_theta, d_eta, d_m_initial, d_s_initial, seq_len, (long long)input_stride,
                    (long long)m_stride, mlpm::make_dims(d, d_hidden)};
    cudaStream_t st = current_stream();
    if (activation == mlpm::ACT_GELU) mlpm::launch_bwd<mlpm::ACT_GELU>(a, batch_size, st);
    else if (activation == mlpm::ACT_SILU) mlpm::launch_bwd<mlpm::ACT_SILU>(a, batch_size, st);
    else mlpm::launch_bwd<mlpm::ACT_RELU>(a, batch_size, st);
}

}  // extern "C"
