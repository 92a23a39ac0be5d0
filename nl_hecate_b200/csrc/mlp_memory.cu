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
    FastDiv div_d, div_h;
};

static Dims make_dims(int d, int dh)
{
    Dims D;
    D.d = d; D.dh = dh;
    D.o1 = dh * d; D.o2 = D.o1 + dh; D.o3 = D.o2 + d * dh; D.ss = D.o3 + d;
    D.div_d = make_fastdiv(d); D.div_h = make_fastdiv(dh);
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

// out(r) = sum_j W[r, j] x[j] for r < R, W row-major [R, C] (shared or global), x in shared
// memory. One warp per row, lanes over columns (coalesced / conflict-free), RB rows in flight per
// warp so that global reads overlap. epi(r, sum) runs on lane 0.
template <int RB, class Epi>
__device__ __forceinline__ void rowdot(const float* __restrict__ W, int R, int C, const float* x, Epi epi)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r0 = warp * RB; r0 < R; r0 += NW * RB) {
        float acc[RB];
#pragma unroll
        for (int u = 0; u < RB; u++) acc[u] = 0.0f;
        for (int j = lane; j < C; j += 32) {
            const float xv = x[j];
#pragma unroll
            for (int u = 0; u < RB; u++)
                if (r0 + u < R) acc[u] = fmaf(W[(size_t)(r0 + u) * C + j], xv, acc[u]);
        }
#pragma unroll
        for (int u = 0; u < RB; u++) {
            const float s = warp_sum(acc[u]);
            if (lane == 0 && r0 + u < R) epi(r0 + u, s);
        }
    }
}

// out(j) = sum_i W[i, j] x[i] for j < C (C <= NT). Thread (g, j) adds rows g, g + G, ... and the G
// partial sums meet in scr[NT]; epi(j, sum) runs on threads j < C. Contains two block barriers;
// every thread of the CTA must call it.
template <class Epi>
__device__ __forceinline__ void colsum(const float* __restrict__ W, int R, int C, const float* x, float* scr,
                                       int g, int j, int G, Epi epi)
{
    float acc = 0.0f;
    if (g < G) {
        int i = g;
        for (; i + 3 * G < R; i += 4 * G) {
            const float w0 = W[(size_t)i * C + j], w1 = W[(size_t)(i + G) * C + j];
            const float w2 = W[(size_t)(i + 2 * G) * C + j], w3 = W[(size_t)(i + 3 * G) * C + j];
            acc = fmaf(w0, x[i], acc); acc = fmaf(w1, x[i + G], acc);
            acc = fmaf(w2, x[i + 2 * G], acc); acc = fmaf(w3, x[i + 3 * G], acc);
        }
        for (; i < R; i += G) acc = fmaf(W[(size_t)i * C + j], x[i], acc);
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

// Element idx of the packed state -> gradient-like outer-product term built from four vectors:
//   W1[r,c] -> a1[r] * x1[c],  b1[r] -> a1[r],  W2[r,c] -> a2[r] * x2[c],  b2[r] -> a2[r]
__device__ __forceinline__ float outer_term(const Dims& D, int idx, const float* a1, const float* x1,
                                            const float* a2, const float* x2)
{
    if (idx < D.o1) { const int r = fd_div(idx, D.div_d); return a1[r] * x1[idx - r * D.d]; }
    if (idx < D.o2) return a1[idx - D.o1];
    if (idx < D.o3) { const int e = idx - D.o2; const int r = fd_div(e, D.div_h); return a2[r] * x2[e - r * D.dh]; }
    return a2[idx - D.o3];
}

struct FwdArgs {
    const float *k, *v, *q, *alpha, *theta, *eta, *m_init, *s_init;
    float *m_states, *s_states, *y;
    int seq_len;
    long long in_stride, m_stride;
    float m_norm_max;
    Dims D;
};

inline size_t fwd_smem_floats(const Dims& D) { return (size_t)((D.ss + 3) & ~3) + 3 * D.d + 3 * D.dh + D.d + NT + 4 * NW; }

template <int ACT, int EPT>
__global__ void __launch_bounds__(NT, 1) mlp_fwd_kernel(FwdArgs a)
{
    extern __shared__ __align__(16) float sm[];
    const Dims& D = a.D;
    const int d = D.d, dh = D.dh, ss = D.ss, tid = threadIdx.x, b = blockIdx.x;
    float* Msm = sm;
    float* kb = Msm + ((ss + 3) & ~3);
    float* vb = kb + d;
    float* qb = vb + d;
    float* pre = qb + d;
    float* h = pre + dh;
    float* gp = h + dh;
    float* e = gp + dh;
    float* scr = e + d;
    float* red = scr + NT;
    const float *W1 = Msm, *b1 = Msm + D.o1, *W2 = Msm + D.o2, *b2 = Msm + D.o3;

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
            Msm[idx] = m; mt[idx] = m; st[idx] = S[i];
        }
    }
    for (int t = 0; t < a.seq_len; t++) {
        for (int i = tid; i < 3 * d; i += NT) {
            const int w = fd_div(i, D.div_d), c = i - w * d;
            kb[i] = (w == 0 ? k : w == 1 ? v : q)[(size_t)t * d + c];     // kb | vb | qb are adjacent
        }
        const float al = alpha[t], th = theta[t], et = eta[t];
        __syncthreads();
        rowdot<2>(W1, dh, d, kb, [&](int r, float s) { const float p = s + b1[r]; pre[r] = p; h[r] = act_fn<ACT>(p); });
        __syncthreads();
        rowdot<2>(W2, d, dh, h, [&](int r, float s) { e[r] = s + b2[r] - vb[r]; });
        __syncthreads();
        colsum(W2, d, dh, e, scr, gh_, jh, Gh, [&](int j, float s) { gp[j] = s * act_prime<ACT>(pre[j]); });
        // S' = eta S - theta grad, M' = (1 - alpha) M + S'
        float* mn = mt + (size_t)(t + 1) * ss;
        float* sn = st + (size_t)(t + 1) * ss;
        float sq[1] = {0.0f};
        const float keep = 1.0f - al;
#pragma unroll
        for (int i = 0; i < EPT; i++) {
            const int idx = tid + i * NT;
            if (idx < ss) {
                const float g = outer_term(D, idx, gp, kb, e, h);
                const float s_new = et * S[i] - th * g;
                const float m_new = fmaf(keep, Msm[idx], s_new);
                S[i] = s_new; Msm[idx] = m_new;
                sn[idx] = s_new;
                if (!clamp) mn[idx] = m_new;
                sq[0] = fmaf(m_new, m_new, sq[0]);
            }
        }
        if (clamp) {      // Frobenius projection over the whole packed state (titans_lmm.rs:812-821)
            block_sum<1>(sq, red);
            const float norm = sqrtf(sq[0]);
            const float scale = norm > a.m_norm_max ? a.m_norm_max / norm : 1.0f;
#pragma unroll
            for (int i = 0; i < EPT; i++) {
                const int idx = tid + i * NT;
                if (idx < ss) { const float m = Msm[idx] * scale; Msm[idx] = m; mn[idx] = m; }
            }
        }
        __syncthreads();
        // y_t = MLP(M_{t+1}, q_t)
        rowdot<2>(W1, dh, d, qb, [&](int r, float s) { pre[r] = act_fn<ACT>(s + b1[r]); });
        __syncthreads();
        rowdot<2>(W2, d, dh, pre, [&](int r, float s) { y[(size_t)t * d + r] = s + b2[r]; });
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

inline size_t bwd_smem_floats(const Dims& D) { return (size_t)((D.ss + 3) & ~3) + 4 * D.d + 8 * D.dh + 3 * D.d + NT + 4 * NW; }

// Reverse loop (titans_lmm.rs:896-1131). Per token, with dM, dS the gradients of M_{t+1}, S_{t+1}:
//   1 readout      pq = W1' q + b1', hq = act(pq); dpq = (W2'^T dy) act'(pq); d_q = W1'^T dpq
//                  dM += {dpq q^T, dpq, dy hq^T, dy}
//   2-4            dS += dM; d_alpha = -<M_t, dM>; d_eta = <S_t, dS>; d_theta = -<grad_t, dS>
//   5 (G = -theta dS)  adj = (G_W1 k + G_b1) act'(pre);  d_err = W2 adj + G_W2 h + G_b2
//                  inj1 = G_W2^T e;  inj0 = G_W1^T gp
//   6              d_v = -d_err;  d_pre = (W2^T d_err + inj1) act'(pre);  d_k = W1^T d_pre + inj0
//                  dM <- (1-alpha) dM + {d_pre k^T, d_pre, d_err h^T + e adj^T, d_err};  dS <- eta dS
// The activation's second derivative does not appear, as in the reference.
template <int ACT, int EPT>
__global__ void __launch_bounds__(NT, 1) mlp_bwd_kernel(BwdArgs a)
{
    extern __shared__ __align__(16) float sm[];
    const Dims& D = a.D;
    const int d = D.d, dh = D.dh, ss = D.ss, tid = threadIdx.x, b = blockIdx.x;
    float* dS = sm;
    float* kb = dS + ((ss + 3) & ~3);     // kb | vb | qb | dyb adjacent
    float* vb = kb + d;
    float* qb = vb + d;
    float* dyb = qb + d;
    float* pre = dyb + d;                 // act'(pre) after the recompute
    float* h = pre + dh;
    float* gp = h + dh;
    float* hq = gp + dh;
    float* dpq = hq + dh;                 // act'(pq), then dpq
    float* adj = dpq + dh;
    float* inj1 = adj + dh;
    float* dpre = inj1 + dh;
    float* e = dpre + dh;
    float* derr = e + d;
    float* inj0 = derr + d;
    float* scr = inj0 + d;
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

    float dM[EPT];
#pragma unroll
    for (int i = 0; i < EPT; i++) {
        dM[i] = 0.0f;
        const int idx = tid + i * NT;
        if (idx < ss) dS[idx] = 0.0f;
    }
    for (int t = a.seq_len - 1; t >= 0; t--) {
        const float* Mt = mt + (size_t)t * ss;
        const float* Mn = Mt + ss;
        const float* St = st + (size_t)t * ss;
        for (int i = tid; i < 4 * d; i += NT) {
            const int w = fd_div(i, D.div_d), c = i - w * d;
            kb[i] = (w == 0 ? k : w == 1 ? v : w == 2 ? q : dy)[(size_t)t * d + c];
        }
        const float al = a.alpha[g0 + t], th = a.theta[g0 + t], et = a.eta[g0 + t];
        __syncthreads();
        // 1: readout through M_{t+1}; 3: the inner gradient's vectors through M_t
        rowdot<8>(Mn, dh, d, qb, [&](int r, float s) { const float p = s + Mn[D.o1 + r]; hq[r] = act_fn<ACT>(p); dpq[r] = act_prime<ACT>(p); });
        rowdot<8>(Mt, dh, d, kb, [&](int r, float s) { const float p = s + Mt[D.o1 + r]; h[r] = act_fn<ACT>(p); pre[r] = act_prime<ACT>(p); });
        __syncthreads();
        rowdot<4>(Mt + D.o2, d, dh, h, [&](int r, float s) { e[r] = s + Mt[D.o3 + r] - vb[r]; });
        colsum(Mn + D.o2, d, dh, dyb, scr, gh_, jh, Gh, [&](int j, float s) { dpq[j] *= s; });
        colsum(Mt + D.o2, d, dh, e, scr, gh_, jh, Gh, [&](int j, float s) { gp[j] = s * pre[j]; });
        colsum(Mn, dh, d, dpq, scr, gd_, jd, Gd, [&](int j, float s) { d_q[(size_t)t * d + j] = s; });
        // dM += readout terms; dS += dM; the three gate gradients
        float acc[3] = {0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < EPT; i++) {
            const int idx = tid + i * NT;
            if (idx < ss) {
                const float dm = dM[i] + outer_term(D, idx, dpq, qb, dyb, hq);
                const float ds = dS[idx] + dm;
                dM[i] = dm; dS[idx] = ds;
                acc[0] = fmaf(Mt[idx], dm, acc[0]);
                acc[1] = fmaf(St[idx], ds, acc[1]);
                acc[2] = fmaf(outer_term(D, idx, gp, kb, e, h), ds, acc[2]);
            }
        }
        block_sum<3>(acc, red);          // its barriers also publish dS
        if (tid == 0) { a.d_alpha[g0 + t] = -acc[0]; a.d_eta[g0 + t] = acc[1]; a.d_theta[g0 + t] = -acc[2]; }
        // 5: products with G = -theta dS
        const float* dS_W1 = dS; const float* dS_b1 = dS + D.o1; const float* dS_W2 = dS + D.o2; const float* dS_b2 = dS + D.o3;
        rowdot<2>(dS_W1, dh, d, kb, [&](int r, float s) { adj[r] = -th * (s + dS_b1[r]) * pre[r]; });
        rowdot<2>(dS_W2, d, dh, h, [&](int r, float s) { derr[r] = -th * (s + dS_b2[r]); });
        colsum(dS_W2, d, dh, e, scr, gh_, jh, Gh, [&](int j, float s) { inj1[j] = -th * s; });
        // (the barriers of colsum published adj and derr)
        rowdot<4>(Mt + D.o2, d, dh, adj, [&](int r, float s) { derr[r] += s; });
        __syncthreads();
        if (tid < d) d_v[(size_t)t * d + tid] = -derr[tid];
        colsum(Mt + D.o2, d, dh, derr, scr, gh_, jh, Gh, [&](int j, float s) { dpre[j] = (s + inj1[j]) * pre[j]; });
        colsum(dS_W1, dh, d, gp, scr, gd_, jd, Gd, [&](int j, float s) { inj0[j] = -th * s; });
        colsum(Mt, dh, d, dpre, scr, gd_, jd, Gd, [&](int j, float s) { d_k[(size_t)t * d + j] = s + inj0[j]; });
        // 6: carry to token t - 1
        const float keep = 1.0f - al;
#pragma unroll
        for (int i = 0; i < EPT; i++) {
            const int idx = tid + i * NT;
            if (idx < ss) {
                float add = outer_term(D, idx, dpre, kb, derr, h);
                if (idx >= D.o2 && idx < D.o3) {          // cross term e adj^T of W2
                    const int el = idx - D.o2, r = fd_div(el, D.div_h);
                    add = fmaf(e[r], adj[el - r * dh], add);
                }
                dM[i] = fmaf(keep, dM[i], add);
                dS[idx] *= et;
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
            atomicAdd(a.d_s_init + idx, dS[idx]);
        }
    }
}

constexpr int EPT_SMALL = 17, EPT_LARGE = 65;     // packed-state elements per thread

static const char* unsupported(int d, int dh)
{
    if (d <= 0 || dh <= 0) return "d and d_hidden must be > 0";
    if (d > NT || dh > NT) return "d and d_hidden above 512 are not supported by the on-chip kernels";
    if ((long long)dh * d * 2 + dh + d > (long long)EPT_LARGE * NT)
        return "packed MLP state above 33280 floats (d = 64, d_hidden = 256) does not fit on one SM";
    return nullptr;
}

template <int ACT>
static bool launch_fwd(const FwdArgs& a, int batch, cudaStream_t st)
{
    const size_t smem = fwd_smem_floats(a.D) * sizeof(float);
    if (a.D.ss <= EPT_SMALL * NT) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(mlp_fwd_kernel<ACT, EPT_SMALL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mlp_fwd_kernel<ACT, EPT_SMALL><<<batch, NT, smem, st>>>(a);
    } else {
        cudaFuncSetAttribute(mlp_fwd_kernel<ACT, EPT_LARGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mlp_fwd_kernel<ACT, EPT_LARGE><<<batch, NT, smem, st>>>(a);
    }
    return check_launch("mlp_fwd_kernel");
}

template <int ACT>
static bool launch_bwd(const BwdArgs& a, int batch, cudaStream_t st)
{
    const size_t smem = bwd_smem_floats(a.D) * sizeof(float);
    if (a.D.ss <= EPT_SMALL * NT) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(mlp_bwd_kernel<ACT, EPT_SMALL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mlp_bwd_kernel<ACT, EPT_SMALL><<<batch, NT, smem, st>>>(a);
    } else {
        cudaFuncSetAttribute(mlp_bwd_kernel<ACT, EPT_LARGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mlp_bwd_kernel<ACT, EPT_LARGE><<<batch, NT, smem, st>>>(a);
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
