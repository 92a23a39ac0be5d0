// Generic-d memory-rule kernels: any head dimension d, every rule (Delta /
// DGD, Titans LMM, Hebbian), every state-emission mode, error clip and
// Frobenius projection. State lives in global memory (L2-resident for small
// d); one CTA per independent problem, rows of the d×d state are owned by
// warps so that the matvec, the rank-1 update and the readout of one token
// need no block barrier between them.
//
// This is the fallback/validation path. The register-resident kernels in
// memory_fast.cuh cover d in {32, 64, 128} without clip/projection.
//
// Math restated from core/src/dispatch.rs:1226-1660 (exact rules) and
// core/kernels/{titans,delta}_chunkwise_{forward,backward}.cu (frozen-M0).
#pragma once

#include "nlh_common.cuh"

namespace nlh {

constexpr int GEN_THREADS = 256;

// Shared-memory floats needed by the generic kernels.
inline size_t gen_fwd_smem(int d) { return (size_t)(4 * d + 32) * sizeof(float); }
inline size_t gen_bwd_smem(int d) { return (size_t)(6 * d + 2 * GEN_THREADS + 32) * sizeof(float); }

// One token of the forward recurrence, executed by the whole CTA.
//   Merr : matrix the prediction error is taken against (current M, or the
//          chunk-start state for the frozen-M0 rule); ignored if ext_err.
//   (Mc,Sc) -> (Mn,Sn) : may alias (in-place).
//   kb,vb,qb : staged token vectors in shared memory (already synchronised).
//   ext_err  : optional pre-computed error vector for this token (phase-2 entries).
// Ends with __syncthreads(): Mn/Sn are visible to the block on return.
template <int RULE>
__device__ __forceinline__ void gen_fwd_token(
    const float* Merr, const float* Mc, const float* Sc, float* Mn, float* Sn,
    const float* kb, const float* vb, const float* qb, float* eb, float* red,
    const float* __restrict__ ext_err,
    float alpha, float theta, float eta, int d, float clip, float mmax, float* y_t)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (RULE != RULE_HEBBIAN) {
        if (ext_err != nullptr) {
            for (int i = threadIdx.x; i < d; i += blockDim.x) eb[i] = ext_err[i];
            __syncthreads();
        } else {
            for (int i = warp; i < d; i += nwarps) {
                const float* row = Merr + (size_t)i * d;
                float p = 0.0f;
                for (int j = lane; j < d; j += 32) p += row[j] * kb[j];
                p = warp_sum(p);
                if (lane == 0) eb[i] = p - vb[i];
            }
            if (clip > 0.0f) {
                __syncthreads();
                float sq = 0.0f;
                for (int i = threadIdx.x; i < d; i += blockDim.x) sq += eb[i] * eb[i];
                float nrm = sqrtf(block_sum(sq, red));
                if (nrm > clip) {
                    float sc = clip / nrm;
                    for (int i = threadIdx.x; i < d; i += blockDim.x) eb[i] *= sc;
                }
                __syncthreads();
            } else {
                __syncwarp();
            }
        }
    }
    const float r = 1.0f - alpha;
    float sq = 0.0f;
    for (int i = warp; i < d; i += nwarps) {
        const float ei = (RULE == RULE_HEBBIAN) ? vb[i] : eb[i];
        const float te = theta * ei;
        for (int j = lane; j < d; j += 32) {
            const size_t idx = (size_t)i * d + j;
            float mn;
            if (RULE == RULE_TITANS) {
                float sn = eta * Sc[idx] - te * kb[j];
                Sn[idx] = sn;
                mn = r * Mc[idx] + sn;
            } else if (RULE == RULE_DELTA) {
                mn = r * Mc[idx] - te * kb[j];
            } else {
                mn = r * Mc[idx] + ei * kb[j];
            }
            Mn[idx] = mn;
            sq += mn * mn;
        }
    }
    if (m_norm_enabled(mmax)) {
        float nrm = sqrtf(block_sum(sq, red));
        if (nrm > mmax) {
            float sc = mmax / nrm;
            for (int i = warp; i < d; i += nwarps)
                for (int j = lane; j < d; j += 32) Mn[(size_t)i * d + j] *= sc;
        }
    }
    if (y_t != nullptr) {
        for (int i = warp; i < d; i += nwarps) {
            const float* row = Mn + (size_t)i * d;
            float s = 0.0f;
            for (int j = lane; j < d; j += 32) s += row[j] * qb[j];
            s = warp_sum(s);
            if (lane == 0) y_t[i] = s;
        }
    }
    __syncthreads();
}

template <int RULE>
__global__ void __launch_bounds__(GEN_THREADS) gen_fwd_kernel(FwdArgs a)
{
    extern __shared__ float sm[];
    const int d = a.d;
    float* kb = sm; float* vb = sm + d; float* qb = sm + 2 * d; float* eb = sm + 3 * d;
    float* red = sm + 4 * d;
    const size_t dd = (size_t)d * d;
    const int b = blockIdx.x;
    const float* k = a.k + (size_t)b * a.in_stride_tok * d;
    const float* v = a.v + (size_t)b * a.in_stride_tok * d;
    const float* q = a.q + (size_t)b * a.in_stride_tok * d;
    const float* alpha = a.alpha + (size_t)b * a.in_stride_tok;
    const float* theta = (RULE != RULE_HEBBIAN) ? a.theta + (size_t)b * a.in_stride_tok : nullptr;
    const float* eta = (RULE == RULE_TITANS) ? a.eta + (size_t)b * a.in_stride_tok : nullptr;
    float* y = a.y + (size_t)b * a.seq_len * d;
    const float* m_init = a.m_init + (size_t)b * a.init_stride;
    const float* s_init = (RULE == RULE_TITANS) ? a.s_init + (size_t)b * a.init_stride : nullptr;
    float* m_out = a.m_out + (size_t)b * a.out_stride;
    float* s_out = (RULE == RULE_TITANS) ? a.s_out + (size_t)b * a.out_stride : nullptr;
    const int mode = a.store_mode;
    float* Mw = (mode == STORE_ALL) ? m_out : a.m_work + (size_t)b * dd;
    float* Sw = nullptr;
    if (RULE == RULE_TITANS) Sw = (mode == STORE_ALL) ? s_out : a.s_work + (size_t)b * dd;

    for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) {
        float m = m_init[idx];
        Mw[idx] = m;
        if (mode == STORE_CKPT) m_out[idx] = m;
        if (RULE == RULE_TITANS) {
            float s = s_init[idx];
            Sw[idx] = s;
            if (mode == STORE_CKPT) s_out[idx] = s;
        }
    }
    __syncthreads();

    int slot = 1;
    const float* M0 = Mw;
    for (int t = 0; t < a.seq_len; t++) {
        if (mode == STORE_CHUNK && (t % a.interval) == 0) {
            const size_t off = (size_t)(t / a.interval) * dd;
            for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) {
                m_out[off + idx] = Mw[idx];
                if (RULE == RULE_TITANS) s_out[off + idx] = Sw[idx];
            }
            M0 = m_out + off;
        }
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            kb[i] = k[(size_t)t * d + i];
            vb[i] = v[(size_t)t * d + i];
            qb[i] = q[(size_t)t * d + i];
        }
        __syncthreads();
        const float* Mc = (mode == STORE_ALL) ? Mw + (size_t)t * dd : Mw;
        float* Mn = (mode == STORE_ALL) ? Mw + (size_t)(t + 1) * dd : Mw;
        const float* Sc = nullptr; float* Sn = nullptr;
        if (RULE == RULE_TITANS) {
            Sc = (mode == STORE_ALL) ? Sw + (size_t)t * dd : Sw;
            Sn = (mode == STORE_ALL) ? Sw + (size_t)(t + 1) * dd : Sw;
        }
        gen_fwd_token<RULE>(a.frozen ? M0 : Mc, Mc, Sc, Mn, Sn, kb, vb, qb, eb, red, nullptr,
                            alpha[t], (RULE != RULE_HEBBIAN) ? theta[t] : 0.0f,
                            (RULE == RULE_TITANS) ? eta[t] : 0.0f, d, a.error_clip, a.m_norm_max,
                            y + (size_t)t * d);
        if (mode == STORE_CKPT && (((t + 1) % a.interval) == 0 || t + 1 == a.seq_len)) {
            const size_t off = (size_t)slot * dd;
            for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) {
                m_out[off + idx] = Mw[idx];
                if (RULE == RULE_TITANS) s_out[off + idx] = Sw[idx];
            }
            slot++;
        }
    }
    if (mode == STORE_CHUNK || mode == STORE_FINAL) {
        const size_t off =
            (mode == STORE_CHUNK) ? (size_t)((a.seq_len + a.interval - 1) / a.interval) * dd : 0;
        for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) {
            m_out[off + idx] = Mw[idx];
            if (RULE == RULE_TITANS) s_out[off + idx] = Sw[idx];
        }
    }
}

// Phase-2 forward for ONE chunk with caller-supplied errors and caller-owned
// running state (core/kernels/titans_phase2_forward.cu, delta_phase2_forward.cu).
template <int RULE>
__global__ void __launch_bounds__(GEN_THREADS) gen_phase2_fwd_kernel(
    const float* __restrict__ k_mem, const float* __restrict__ q_mem,
    const float* __restrict__ alpha_g, const float* __restrict__ theta_g,
    const float* __restrict__ eta_g, const float* __restrict__ errors,
    float* m_work, float* s_work, float* m_chunk_states, float* s_chunk_states, float* y_g,
    int seq_len, int d, int chunk_size, int chunk_idx, float m_norm_max)
{
    extern __shared__ float sm[];
    float* kb = sm; float* vb = sm + d; float* qb = sm + 2 * d; float* eb = sm + 3 * d;
    float* red = sm + 4 * d;
    const size_t dd = (size_t)d * d;
    const int b = blockIdx.x;
    const int nc = (seq_len + chunk_size - 1) / chunk_size;
    const int t0 = chunk_idx * chunk_size;
    const int t1 = min(t0 + chunk_size, seq_len);
    const float* k = k_mem + (size_t)b * seq_len * d;
    const float* q = q_mem + (size_t)b * seq_len * d;
    const float* alpha = alpha_g + (size_t)b * seq_len;
    const float* theta = theta_g + (size_t)b * seq_len;
    const float* eta = (RULE == RULE_TITANS) ? eta_g + (size_t)b * seq_len : nullptr;
    const float* err = errors + (size_t)b * chunk_size * d;
    float* Mw = m_work + (size_t)b * dd;
    float* Sw = (RULE == RULE_TITANS) ? s_work + (size_t)b * dd : nullptr;
    float* mcs = m_chunk_states + (size_t)b * (nc + 1) * dd;
    float* scs = (RULE == RULE_TITANS) ? s_chunk_states + (size_t)b * (nc + 1) * dd : nullptr;
    float* y = y_g + (size_t)b * seq_len * d;

    for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) {
        mcs[(size_t)chunk_idx * dd + idx] = Mw[idx];
        if (RULE == RULE_TITANS) scs[(size_t)chunk_idx * dd + idx] = Sw[idx];
    }
    __syncthreads();
    for (int t = t0; t < t1; t++) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            kb[i] = k[(size_t)t * d + i];
            vb[i] = 0.0f;
            qb[i] = q[(size_t)t * d + i];
        }
        __syncthreads();
        gen_fwd_token<RULE>(Mw, Mw, Sw, Mw, Sw, kb, vb, qb, eb, red, err + (size_t)(t - t0) * d,
                            alpha[t], theta[t], (RULE == RULE_TITANS) ? eta[t] : 0.0f, d, 0.0f,
                            m_norm_max, y + (size_t)t * d);
    }
    if (chunk_idx == nc - 1) {
        for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) {
            mcs[(size_t)nc * dd + idx] = Mw[idx];
            if (RULE == RULE_TITANS) scs[(size_t)nc * dd + idx] = Sw[idx];
        }
    }
}

// One token of the reverse pass, executed by the whole CTA, in the order of operations of the
// reference's rust_{titans,delta,hebbian}_backward (core/src/dispatch.rs:1300-1660). d_M/d_S live in
// global work buffers owned (by row) by warps.
template <int RULE, bool FROZEN>
__device__ __forceinline__ void gen_bwd_token(
    const float* __restrict__ Mt, const float* __restrict__ Mn, const float* __restrict__ St,
    const float* __restrict__ M0, float* dM, float* dS, float* dM0,
    const float* __restrict__ k_t, const float* __restrict__ v_t, const float* __restrict__ q_t,
    const float* __restrict__ dy_t, const float* __restrict__ ext_err,
    float* sm, float alpha, float theta, float eta, int d, float clip,
    float* dk_t, float* dv_t, float* dq_t, float* dalpha_t, float* dtheta_t, float* deta_t)
{
    float* kb = sm; float* vb = sm + d; float* qb = sm + 2 * d; float* dyb = sm + 3 * d;
    float* eb = sm + 4 * d; float* ub = sm + 5 * d;
    float* part = sm + 6 * d;                 // [2 * GEN_THREADS]
    float* red = part + 2 * GEN_THREADS;      // [32]
    const int tid = threadIdx.x, nt = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;

    for (int i = tid; i < d; i += nt) {
        kb[i] = k_t[i];
        vb[i] = (v_t != nullptr) ? v_t[i] : 0.0f;
        qb[i] = q_t[i];
        dyb[i] = dy_t[i];
    }
    __syncthreads();

    // ── row pass ──
    float acc_a = 0.0f, acc_e = 0.0f;
    for (int i = warp; i < d; i += nwarps) {
        const float dyi = dyb[i];
        float p = 0.0f, u = 0.0f;
        for (int j = lane; j < d; j += 32) {
            const size_t idx = (size_t)i * d + j;
            const float mt = Mt[idx];
            const float dm = dM[idx] + dyi * qb[j];
            dM[idx] = dm;
            float g = dm;
            if (RULE == RULE_TITANS) {
                const float ds = dS[idx] + dm;
                dS[idx] = ds;
                g = ds;
                acc_e += St[idx] * ds;
            }
            acc_a += mt * dm;
            if (RULE != RULE_HEBBIAN) p += (FROZEN ? M0[idx] : mt) * kb[j];
            u += g * kb[j];
        }
        p = warp_sum(p);
        u = warp_sum(u);
        if (lane == 0) {
            if (RULE != RULE_HEBBIAN) eb[i] = (ext_err != nullptr) ? ext_err[i] : (p - vb[i]);
            ub[i] = u;
        }
    }
    __syncthreads();
    if (RULE != RULE_HEBBIAN && clip > 0.0f && ext_err == nullptr) {
        float sq = 0.0f;
        for (int i = tid; i < d; i += nt) sq += eb[i] * eb[i];
        float nrm = sqrtf(block_sum(sq, red));
        if (nrm > clip) {
            float sc = clip / nrm;
            for (int i = tid; i < d; i += nt) eb[i] *= sc;
        }
        __syncthreads();
    }
    // ── per-token scalars ──
    const float da = block_sum(acc_a, red);
    float de = 0.0f, dth = 0.0f;
    if (RULE == RULE_TITANS) de = block_sum(acc_e, red);
    if (RULE != RULE_HEBBIAN) {
        float s = 0.0f;
        for (int i = tid; i < d; i += nt) s += eb[i] * ub[i];
        dth = block_sum(s, red);
    }
    if (tid == 0) {
        *dalpha_t = -da;
        if (RULE == RULE_TITANS) *deta_t = de;
        if (RULE != RULE_HEBBIAN) *dtheta_t = -dth;
    }
    for (int i = tid; i < d; i += nt)
        dv_t[i] = (RULE == RULE_HEBBIAN) ? ub[i] : theta * ub[i];   // d_v = -d_err = theta * (G k)

    // ── column pass: d_q = M_{t+1}^T d_y ; d_k = -theta G^T e + Mk^T d_err ──
    const float* G = (RULE == RULE_TITANS) ? dS : dM;
    const float* Mk = FROZEN ? M0 : Mt;
    if (d <= nt) {
        const int ngroups = nt / d;
        const int g = tid / d, j = tid - g * d;
        if (g < ngroups) {
            float sq = 0.0f, sk = 0.0f;
            for (int i = g; i < d; i += ngroups) {
                const size_t idx = (size_t)i * d + j;
                sq += Mn[idx] * dyb[i];
                if (RULE == RULE_HEBBIAN) {
                    sk += dM[idx] * vb[i];
                } else {
                    const float dei = -theta * ub[i];
                    sk += (-theta * G[idx]) * eb[i] + Mk[idx] * dei;
                }
            }
            part[g * d + j] = sq;
            part[GEN_THREADS + g * d + j] = sk;
        }
        __syncthreads();
        if (tid < d) {
            float sq = 0.0f, sk = 0.0f;
            for (int gg = 0; gg < ngroups; gg++) {
                sq += part[gg * d + tid];
                sk += part[GEN_THREADS + gg * d + tid];
            }
            dq_t[tid] = sq;
            dk_t[tid] = sk;
        }
    } else {
        for (int j = tid; j < d; j += nt) {
            float sq = 0.0f, sk = 0.0f;
            for (int i = 0; i < d; i++) {
                const size_t idx = (size_t)i * d + j;
                sq += Mn[idx] * dyb[i];
                if (RULE == RULE_HEBBIAN) {
                    sk += dM[idx] * vb[i];
                } else {
                    const float dei = -theta * ub[i];
                    sk += (-theta * G[idx]) * eb[i] + Mk[idx] * dei;
                }
            }
            dq_t[j] = sq;
            dk_t[j] = sk;
        }
    }
    __syncthreads();

    // ── propagate d_M, d_S to the previous token ──
    const float r = 1.0f - alpha;
    for (int i = warp; i < d; i += nwarps) {
        const float dei = (RULE == RULE_HEBBIAN) ? 0.0f : -theta * ub[i];
        for (int j = lane; j < d; j += 32) {
            const size_t idx = (size_t)i * d + j;
            if (RULE == RULE_TITANS) dS[idx] = eta * dS[idx];
            float dm = r * dM[idx];
            if (RULE != RULE_HEBBIAN) {
                const float o = dei * kb[j];
                if (FROZEN) dM0[idx] += o; else dm += o;
            }
            dM[idx] = dm;
        }
    }
    __syncthreads();
}

template <int RULE>
__global__ void __launch_bounds__(GEN_THREADS) gen_bwd_kernel(BwdArgs a)
{
    extern __shared__ float sm[];
    const int d = a.d;
    const size_t dd = (size_t)d * d;
    const int b = blockIdx.x;
    const size_t so = (size_t)b * a.seq_len * d, go = (size_t)b * a.seq_len;
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
    const float* straj = (RULE == RULE_TITANS) ? a.s_traj + (size_t)b * a.traj_stride : nullptr;
    float* dM = a.dM + (size_t)b * dd;
    float* dS = (RULE == RULE_TITANS) ? a.dS + (size_t)b * dd : nullptr;

    for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) {
        dM[idx] = a.d_m_seed ? a.d_m_seed[(size_t)b * dd + idx] : 0.0f;
        if (RULE == RULE_TITANS) dS[idx] = a.d_s_seed ? a.d_s_seed[(size_t)b * dd + idx] : 0.0f;
    }
    __syncthreads();

    if (a.chunk <= 0) {
        for (int t = a.t_end - 1; t >= a.t_start; t--) {
            const size_t lt = (size_t)(t - a.t_start);
            gen_bwd_token<RULE, false>(
                mtraj + lt * dd, mtraj + (lt + 1) * dd,
                (RULE == RULE_TITANS) ? straj + lt * dd : nullptr, nullptr, dM, dS, nullptr,
                k + (size_t)t * d, v + (size_t)t * d, q + (size_t)t * d, dy + (size_t)t * d, nullptr,
                sm, alpha[t], (RULE != RULE_HEBBIAN) ? theta[t] : 0.0f,
                (RULE == RULE_TITANS) ? eta[t] : 0.0f, d, a.error_clip,
                dk + (size_t)t * d, dv + (size_t)t * d, dq + (size_t)t * d, dalpha + t,
                (RULE != RULE_HEBBIAN) ? dtheta + t : nullptr,
                (RULE == RULE_TITANS) ? deta + t : nullptr);
        }
    } else {
        // Boundary states every a.chunk tokens (chunk-start states of the frozen-M0
        // rule, or checkpoints of the exact rule): recompute the trajectory of one
        // chunk into m_rec/s_rec, then walk it in reverse.
        const bool frozen = a.frozen != 0;
        float* dM0 = frozen ? a.dM0 + (size_t)b * dd : nullptr;
        float* mrec = a.m_rec + (size_t)b * (a.chunk + 1) * dd;
        float* srec = (RULE == RULE_TITANS) ? a.s_rec + (size_t)b * (a.chunk + 1) * dd : nullptr;
        float* kb = sm; float* vb = sm + d; float* qb = sm + 2 * d; float* eb = sm + 4 * d;
        float* red = sm + 6 * d + 2 * GEN_THREADS;
        const int nc = (a.seq_len + a.chunk - 1) / a.chunk;
        for (int c = nc - 1; c >= 0; c--) {
            const int t0 = c * a.chunk;
            const int t1 = min(t0 + a.chunk, a.seq_len);
            for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) {
                mrec[idx] = mtraj[(size_t)c * dd + idx];
                if (RULE == RULE_TITANS) srec[idx] = straj[(size_t)c * dd + idx];
                if (frozen) dM0[idx] = 0.0f;
            }
            __syncthreads();
            for (int t = t0; t < t1; t++) {
                const size_t tl = (size_t)(t - t0);
                for (int i = threadIdx.x; i < d; i += blockDim.x) {
                    kb[i] = k[(size_t)t * d + i];
                    vb[i] = v[(size_t)t * d + i];
                    qb[i] = 0.0f;
                }
                __syncthreads();
                gen_fwd_token<RULE>(frozen ? mrec : mrec + tl * dd, mrec + tl * dd,
                                    (RULE == RULE_TITANS) ? srec + tl * dd : nullptr,
                                    mrec + (tl + 1) * dd,
                                    (RULE == RULE_TITANS) ? srec + (tl + 1) * dd : nullptr,
                                    kb, vb, qb, eb, red, nullptr, alpha[t],
                                    (RULE != RULE_HEBBIAN) ? theta[t] : 0.0f,
                                    (RULE == RULE_TITANS) ? eta[t] : 0.0f, d, a.error_clip,
                                    a.m_norm_max, nullptr);
            }
            for (int t = t1 - 1; t >= t0; t--) {
                const size_t tl = (size_t)(t - t0);
                const float* Mt = mrec + tl * dd;
                const float* Mn = mrec + (tl + 1) * dd;
                const float* St = (RULE == RULE_TITANS) ? srec + tl * dd : nullptr;
                const float th = (RULE != RULE_HEBBIAN) ? theta[t] : 0.0f;
                const float et = (RULE == RULE_TITANS) ? eta[t] : 0.0f;
                float* dth_t = (RULE != RULE_HEBBIAN) ? dtheta + t : nullptr;
                float* det_t = (RULE == RULE_TITANS) ? deta + t : nullptr;
                if (frozen)
                    gen_bwd_token<RULE, true>(Mt, Mn, St, mrec, dM, dS, dM0, k + (size_t)t * d,
                        v + (size_t)t * d, q + (size_t)t * d, dy + (size_t)t * d, nullptr, sm,
                        alpha[t], th, et, d, a.error_clip, dk + (size_t)t * d, dv + (size_t)t * d,
                        dq + (size_t)t * d, dalpha + t, dth_t, det_t);
                else
                    gen_bwd_token<RULE, false>(Mt, Mn, St, nullptr, dM, dS, nullptr,
                        k + (size_t)t * d, v + (size_t)t * d, q + (size_t)t * d,
                        dy + (size_t)t * d, nullptr, sm, alpha[t], th, et, d, a.error_clip,
                        dk + (size_t)t * d, dv + (size_t)t * d, dq + (size_t)t * d, dalpha + t,
                        dth_t, det_t);
            }
            if (frozen) {
                for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) dM[idx] += dM0[idx];
                __syncthreads();
            }
        }
    }

    if (a.d_m_out == nullptr) return;   // initial-state gradients not requested
    for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) {
        if (a.atomic_out) {
            atomicAdd(&a.d_m_out[idx], dM[idx]);
            if (RULE == RULE_TITANS) atomicAdd(&a.d_s_out[idx], dS[idx]);
        } else {
            a.d_m_out[(size_t)b * dd + idx] = dM[idx];
            if (RULE == RULE_TITANS) a.d_s_out[(size_t)b * dd + idx] = dS[idx];
        }
    }
}

// Phase-2 backward for ONE chunk: caller-supplied errors, caller-owned running
// d_M/d_S (persist across the per-chunk calls), d_M0 and recompute buffers
// (core/kernels/titans_phase2_backward.cu, delta_phase2_backward.cu).
template <int RULE>
__global__ void __launch_bounds__(GEN_THREADS) gen_phase2_bwd_kernel(
    const float* __restrict__ k_mem, const float* __restrict__ q_mem,
    const float* __restrict__ alpha_g, const float* __restrict__ theta_g,
    const float* __restrict__ eta_g, const float* __restrict__ errors,
    const float* __restrict__ m_chunk_states, const float* __restrict__ s_chunk_states,
    const float* __restrict__ d_y, float* d_k, float* d_v, float* d_q,
    float* d_alpha, float* d_theta, float* d_eta,
    float* dM_g, float* dS_g, float* dM0_g, float* m_rec_g, float* s_rec_g,
    int seq_len, int d, int chunk_size, int chunk_idx, float m_norm_max)
{
    extern __shared__ float sm[];
    const size_t dd = (size_t)d * d;
    const int b = blockIdx.x;
    const int nc = (seq_len + chunk_size - 1) / chunk_size;
    const int t0 = chunk_idx * chunk_size;
    const int t1 = min(t0 + chunk_size, seq_len);
    const size_t so = (size_t)b * seq_len * d, go = (size_t)b * seq_len;
    const float* k = k_mem + so; const float* q = q_mem + so; const float* dy = d_y + so;
    const float* alpha = alpha_g + go; const float* theta = theta_g + go;
    const float* eta = (RULE == RULE_TITANS) ? eta_g + go : nullptr;
    const float* err = errors + (size_t)b * chunk_size * d;
    const float* mcs = m_chunk_states + (size_t)b * (nc + 1) * dd;
    const float* scs = (RULE == RULE_TITANS) ? s_chunk_states + (size_t)b * (nc + 1) * dd : nullptr;
    float* dM = dM_g + (size_t)b * dd;
    float* dS = (RULE == RULE_TITANS) ? dS_g + (size_t)b * dd : nullptr;
    float* dM0 = dM0_g + (size_t)b * dd;
    float* mrec = m_rec_g + (size_t)b * (chunk_size + 1) * dd;
    float* srec = (RULE == RULE_TITANS) ? s_rec_g + (size_t)b * (chunk_size + 1) * dd : nullptr;
    float* kb = sm; float* vb = sm + d; float* qb = sm + 2 * d; float* eb = sm + 4 * d;
    float* red = sm + 6 * d + 2 * GEN_THREADS;

    for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) {
        mrec[idx] = mcs[(size_t)chunk_idx * dd + idx];
        if (RULE == RULE_TITANS) srec[idx] = scs[(size_t)chunk_idx * dd + idx];
        dM0[idx] = 0.0f;
    }
    __syncthreads();
    for (int t = t0; t < t1; t++) {
        const size_t tl = (size_t)(t - t0);
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            kb[i] = k[(size_t)t * d + i]; vb[i] = 0.0f; qb[i] = 0.0f;
        }
        __syncthreads();
        gen_fwd_token<RULE>(mrec, mrec + tl * dd, (RULE == RULE_TITANS) ? srec + tl * dd : nullptr,
                            mrec + (tl + 1) * dd,
                            (RULE == RULE_TITANS) ? srec + (tl + 1) * dd : nullptr,
                            kb, vb, qb, eb, red, err + tl * d, alpha[t], theta[t],
                            (RULE == RULE_TITANS) ? eta[t] : 0.0f, d, 0.0f, m_norm_max, nullptr);
    }
    for (int t = t1 - 1; t >= t0; t--) {
        const size_t tl = (size_t)(t - t0);
        gen_bwd_token<RULE, true>(
            mrec + tl * dd, mrec + (tl + 1) * dd, (RULE == RULE_TITANS) ? srec + tl * dd : nullptr,
            mrec, dM, dS, dM0, k + (size_t)t * d, nullptr, q + (size_t)t * d, dy + (size_t)t * d,
            err + tl * d, sm, alpha[t], theta[t], (RULE == RULE_TITANS) ? eta[t] : 0.0f, d, 0.0f,
            d_k + so + (size_t)t * d, d_v + so + (size_t)t * d, d_q + so + (size_t)t * d,
            d_alpha + go + t, d_theta + go + t, (RULE == RULE_TITANS) ? d_eta + go + t : nullptr);
    }
    for (size_t idx = threadIdx.x; idx < dd; idx += blockDim.x) dM[idx] += dM0[idx];
}

// predictions[row,:] -= v[row,:]; optional per-row L2 clip
// (core/kernels/error_subtract_clip.cu). One warp per row.
static __global__ void error_subtract_clip_kernel(float* pred, const float* __restrict__ v,
                                           int rows, int d, float clip)
{
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    float* p = pred + (size_t)row * d;
    const float* vr = v + (size_t)row * d;
    float sq = 0.0f;
    for (int j = lane; j < d; j += 32) {
        float e = p[j] - vr[j];
        p[j] = e;
        sq += e * e;
    }
    if (clip > 0.0f) {
        float nrm = sqrtf(warp_sum(sq));
        if (nrm > clip) {
            float sc = clip / nrm;
            for (int j = lane; j < d; j += 32) p[j] *= sc;
        }
    }
}

// Frobenius clamp of each d×d matrix in a batch (core/kernels/m_norm_clamp.cu).
static __global__ void __launch_bounds__(GEN_THREADS) m_norm_clamp_kernel(float* m, size_t dd, float mmax)
{
    __shared__ float red[32];
    float* mb = m + (size_t)blockIdx.x * dd;
    float sq = 0.0f;
    for (size_t i = threadIdx.x; i < dd; i += blockDim.x) sq += mb[i] * mb[i];
    float nrm = sqrtf(block_sum(sq, red));
    if (nrm > mmax) {
        float sc = mmax / nrm;
        for (size_t i = threadIdx.x; i < dd; i += blockDim.x) mb[i] *= sc;
    }
}

}  // namespace nlh
