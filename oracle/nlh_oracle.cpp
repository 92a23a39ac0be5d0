// CPU oracle for the NL_Hecate memory-rule / SWA / AdamW hot path.
//
// TEST INFRASTRUCTURE ONLY. This file is a plain-loop CPU restatement of the
// reference's Rust (and, where no Rust statement exists, CUDA) algorithms. It
// is the checker the CUDA kernels are compared against and the CPU arm of the
// benchmark; nothing in the product path may link or call it.
//
// Parity pin: the reference is a Rust workspace and cannot be compiled in the
// build environment, and it ships no golden vectors. The oracle is pinned by
// (i) the reference's own known-answer unit tests re-created in the test
// suite (SWA window/causal cases, sigmoid/softplus values, EMA step identity,
// SimpleRng determinism/range), (ii) central finite differences with the
// reference's eps/tolerances, (iii) the chunk_size=1 == per-token identity.
// There are no reference-run fixtures: "parity pinned by known-answer tests
// and identities, not by reference outputs".
//
// Every function cites the reference file:line it restates. Single-threaded
// per problem like the Rust code; `*_batched_mt` entries only fan independent
// problems over host threads for the timed CPU baseline.
//
// Build: g++ -O2 -ffp-contract=off -fPIC -shared (see oracle/Makefile).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>
#include <algorithm>
#include <limits>

#define ORC_API extern "C" __attribute__((visibility("default")))

// ───────────────────────── SimpleRng (core/src/tensor.rs:380-408) ─────────
struct SimpleRng {
    uint64_t state;
    explicit SimpleRng(uint64_t seed) : state(seed == 0 ? 1 : seed) {}
    uint64_t next_u64() {
        state ^= state << 13;
        state ^= state >> 7;
        state ^= state << 17;
        return state;
    }
    float uniform(float scale) {
        // (next as f64) / (u64::MAX as f64), then 2*(u as f32) - 1 in f32.
        double u = (double)next_u64() / 18446744073709551615.0;
        float uf = (float)u;
        return (2.0f * uf - 1.0f) * scale;
    }
};

ORC_API void orc_rng_fill_uniform(uint64_t seed, float scale, float* out, int64_t n) {
    SimpleRng rng(seed);
    for (int64_t i = 0; i < n; i++) out[i] = rng.uniform(scale);
}

// Sequential draws from ONE generator into several buffers is how the
// reference initialises parameter structs; expose a stateful handle.
ORC_API void orc_rng_stream(uint64_t* state_io, float scale, float* out, int64_t n) {
    SimpleRng rng(1);
    rng.state = *state_io == 0 ? 1 : *state_io;
    for (int64_t i = 0; i < n; i++) out[i] = rng.uniform(scale);
    *state_io = rng.state;
}

// Token ids: rng.next_u64() % vocab (core/src/traced_forward.rs:1549-1554).
ORC_API void orc_rng_tokens(uint64_t seed, uint64_t vocab, int64_t* out, int64_t n) {
    SimpleRng rng(seed);
    for (int64_t i = 0; i < n; i++) out[i] = (int64_t)(rng.next_u64() % vocab);
}

ORC_API uint64_t orc_rng_next_u64(uint64_t* state_io) {
    SimpleRng rng(1);
    rng.state = *state_io == 0 ? 1 : *state_io;
    uint64_t v = rng.next_u64();
    *state_io = rng.state;
    return v;
}

// ───────────────────────── scalar helpers (core/src/tensor.rs:199-227) ────
static inline float sigmoid_f32(float x) {
    if (x >= 15.0f) return 1.0f;
    if (x <= -15.0f) return 0.0f;
    return 1.0f / (1.0f + std::exp(-x));
}
static inline float softplus_f32(float x) {
    if (x >= 15.0f) return x;
    if (x <= -15.0f) return 0.0f;
    return std::log(1.0f + std::exp(x));
}
ORC_API float orc_sigmoid(float x) { return sigmoid_f32(x); }
ORC_API float orc_softplus(float x) { return softplus_f32(x); }

// bf16 round-to-nearest-even of an f32 (core/src/bf16.rs:16-28).
static inline float bf16_round(float x) {
    uint32_t bits;
    std::memcpy(&bits, &x, 4);
    if (x != x) {  // NaN → quiet NaN, sign kept
        uint32_t t = ((bits & 0x80000000u) | 0x7FC00000u);
        float r; std::memcpy(&r, &t, 4); return r;
    }
    uint32_t rounding_bias = 0x7FFFu + ((bits >> 16) & 1u);
    bits += rounding_bias;  // wrapping add
    bits &= 0xFFFF0000u;
    float r; std::memcpy(&r, &bits, 4); return r;
}
ORC_API void orc_bf16_round(const float* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = bf16_round(in[i]);
}

// L2 row normalisation (core/src/tensor.rs:296-314) and its backward (:320-351).
ORC_API void orc_l2_normalize_rows(float* x, float* norms, int64_t n_rows, int64_t d) {
    const float eps = 1e-8f;
    for (int64_t i = 0; i < n_rows; i++) {
        float* row = x + i * d;
        float sq = 0.0f;
        for (int64_t j = 0; j < d; j++) sq += row[j] * row[j];
        float norm = std::sqrt(sq);
        norms[i] = norm;
        float inv = 1.0f / std::max(norm, eps);
        for (int64_t j = 0; j < d; j++) row[j] *= inv;
    }
}
ORC_API void orc_l2_normalize_rows_backward(const float* d_out, const float* x_norm,
                                            const float* norms, float* d_in,
                                            int64_t n_rows, int64_t d) {
    const float eps = 1e-8f;
    for (int64_t i = 0; i < n_rows; i++) {
        const float* go = d_out + i * d;
        const float* xn = x_norm + i * d;
        float* gi = d_in + i * d;
        if (norms[i] >= eps) {
            float inv = 1.0f / norms[i];
            float dot = 0.0f;
            for (int64_t j = 0; j < d; j++) dot += go[j] * xn[j];
            for (int64_t j = 0; j < d; j++) gi[j] = (go[j] - xn[j] * dot) * inv;
        } else {
            float inv_eps = 1.0f / eps;
            for (int64_t j = 0; j < d; j++) gi[j] = go[j] * inv_eps;
        }
    }
}

// ───────────────────────── clip / clamp (core/src/dispatch.rs:1226-1244) ──
static void clip_error_l2(float* e, int d, float clip) {
    if (clip <= 0.0f) return;
    float nsq = 0.0f;
    for (int i = 0; i < d; i++) nsq += e[i] * e[i];
    float norm = std::sqrt(nsq);
    if (norm > clip) {
        float s = clip / norm;
        for (int i = 0; i < d; i++) e[i] *= s;
    }
}
static void clamp_m_norm(float* m, int64_t dd, float m_norm_max) {
    if (m_norm_max > 0.0f && m_norm_max < std::numeric_limits<float>::max()) {
        float nsq = 0.0f;
        for (int64_t i = 0; i < dd; i++) nsq += m[i] * m[i];
        float norm = std::sqrt(nsq);
        if (norm > m_norm_max) {
            float s = m_norm_max / norm;
            for (int64_t i = 0; i < dd; i++) m[i] *= s;
        }
    }
}
ORC_API void orc_m_norm_clamp(float* m, int d, int batch, float m_norm_max) {
    // core/kernels/m_norm_clamp.cu: disabled when max <= 0 or >= 1e30.
    if (m_norm_max <= 0.0f || m_norm_max >= 1e30f) return;
    for (int b = 0; b < batch; b++) clamp_m_norm(m + (int64_t)b * d * d, (int64_t)d * d, m_norm_max);
}

// ───────────────────────── Delta rule (core/src/dispatch.rs:1247-1389) ────
ORC_API void orc_delta_forward(const float* k_mem, const float* v_mem, const float* q_mem,
                               const float* alpha, const float* theta, const float* m_initial,
                               float* m_states, float* y, int seq_len, int d,
                               float error_clip, float m_norm_max) {
    const int64_t dd = (int64_t)d * d;
    std::memcpy(m_states, m_initial, dd * sizeof(float));
    std::vector<float> pred(d), err(d);
    for (int t = 0; t < seq_len; t++) {
        const float* k_t = k_mem + (int64_t)t * d;
        const float* v_t = v_mem + (int64_t)t * d;
        const float* q_t = q_mem + (int64_t)t * d;
        const float* m_t = m_states + (int64_t)t * dd;
        float* m_n = m_states + (int64_t)(t + 1) * dd;
        for (int i = 0; i < d; i++) {
            float s = 0.0f;
            for (int j = 0; j < d; j++) s += m_t[i * d + j] * k_t[j];
            pred[i] = s;
        }
        for (int i = 0; i < d; i++) err[i] = pred[i] - v_t[i];
        clip_error_l2(err.data(), d, error_clip);
        float ret = 1.0f - alpha[t];
        float th = theta[t];
        for (int i = 0; i < d; i++)
            for (int j = 0; j < d; j++)
                m_n[i * d + j] = ret * m_t[i * d + j] - th * err[i] * k_t[j];
        clamp_m_norm(m_n, dd, m_norm_max);
        for (int i = 0; i < d; i++) {
            float s = 0.0f;
            for (int j = 0; j < d; j++) s += m_n[i * d + j] * q_t[j];
            y[(int64_t)t * d + i] = s;
        }
    }
}

// Segment form: reverse loop over [0, seq_len) seeded with d_m_seed (may be
// null = zeros), writing d_m_out. The full backward is the seed=0 case.
// Segment semantics: core/kernels/delta_backward.cu (segment kernel),
// core/src/cuda_ffi.rs:221-282.
ORC_API void orc_delta_backward(const float* k_mem, const float* v_mem, const float* q_mem,
                                const float* alpha, const float* theta, const float* m_states,
                                const float* d_y, const float* d_m_seed,
                                float* d_k, float* d_v, float* d_q,
                                float* d_alpha, float* d_theta, float* d_m_out,
                                int seq_len, int d, float error_clip) {
    const int64_t dd = (int64_t)d * d;
    std::vector<float> dM(dd, 0.0f), pred(d), err(d), derr(d);
    if (d_m_seed) std::memcpy(dM.data(), d_m_seed, dd * sizeof(float));
    for (int t = seq_len - 1; t >= 0; t--) {
        const float* k_t = k_mem + (int64_t)t * d;
        const float* v_t = v_mem + (int64_t)t * d;
        const float* q_t = q_mem + (int64_t)t * d;
        const float* dy = d_y + (int64_t)t * d;
        const float* m_t = m_states + (int64_t)t * dd;
        const float* m_n = m_states + (int64_t)(t + 1) * dd;
        float th = theta[t];
        for (int i = 0; i < d; i++)
            for (int j = 0; j < d; j++) dM[i * d + j] += dy[i] * q_t[j];
        for (int j = 0; j < d; j++) {
            float s = 0.0f;
            for (int i = 0; i < d; i++) s += m_n[i * d + j] * dy[i];
            d_q[(int64_t)t * d + j] = s;
        }
        for (int i = 0; i < d; i++) {
            float s = 0.0f;
            for (int j = 0; j < d; j++) s += m_t[i * d + j] * k_t[j];
            pred[i] = s;
        }
        for (int i = 0; i < d; i++) err[i] = pred[i] - v_t[i];
        clip_error_l2(err.data(), d, error_clip);
        float da = 0.0f, dt = 0.0f;
        for (int i = 0; i < d; i++)
            for (int j = 0; j < d; j++) {
                da += m_t[i * d + j] * dM[i * d + j];
                dt += err[i] * k_t[j] * dM[i * d + j];
            }
        d_alpha[t] = -da;
        d_theta[t] = -dt;
        for (int i = 0; i < d; i++) {
            float s = 0.0f;
            for (int j = 0; j < d; j++) s += (-th * dM[i * d + j]) * k_t[j];
            derr[i] = s;
        }
        for (int j = 0; j < d; j++) {
            float s = 0.0f;
            for (int i = 0; i < d; i++) s += (-th * dM[i * d + j]) * err[i];
            d_k[(int64_t)t * d + j] = s;
        }
        for (int j = 0; j < d; j++) {
            float s = 0.0f;
            for (int i = 0; i < d; i++) s += m_t[i * d + j] * derr[i];
            d_k[(int64_t)t * d + j] += s;
        }
        for (int i = 0; i < d; i++) d_v[(int64_t)t * d + i] = -derr[i];
        float ret = 1.0f - alpha[t];
        for (int i = 0; i < d; i++)
            for (int j = 0; j < d; j++)
                dM[i * d + j] = ret * dM[i * d + j] + derr[i] * k_t[j];
    }
    std::memcpy(d_m_out, dM.data(), dd * sizeof(float));
}

// ───────────────────────── Titans LMM (core/src/dispatch.rs:1392-1563) ────
ORC_API void orc_titans_forward(const float* k_mem, const float* v_mem, const float* q_mem,
                                const float* alpha, const float* theta, const float* eta,
                                const float* m_initial, const float* s_initial,
                                float* m_states, float* s_states, float* y,
                                int seq_len, int d, float error_clip, float m_norm_max) {
    const int64_t dd = (int64_t)d * d;
    std::memcpy(m_states, m_initial, dd * sizeof(float));
    std::memcpy(s_states, s_initial, dd * sizeof(float));
    std::vector<float> pred(d), err(d);
    for (int t = 0; t < seq_len; t++) {
        const float* k_t = k_mem + (int64_t)t * d;
        const float* v_t = v_mem + (int64_t)t * d;
        const float* q_t = q_mem + (int64_t)t * d;
        const float* m_t = m_states + (int64_t)t * dd;
        float* m_n = m_states + (int64_t)(t + 1) * dd;
        const float* s_t = s_states + (int64_t)t * dd;
        float* s_n = s_states + (int64_t)(t + 1) * dd;
        for (int i = 0; i < d; i++) {
            float s = 0.0f;
            for (int j = 0; j < d; j++) s += m_t[i * d + j] * k_t[j];
            pred[i] = s;
        }
        for (int i = 0; i < d; i++) err[i] = pred[i] - v_t[i];
        clip_error_l2(err.data(), d, error_clip);
        float et = eta[t], th = theta[t];
        for (int i = 0; i < d; i++)
            for (int j = 0; j < d; j++)
                s_n[i * d + j] = et * s_t[i * d + j] - th * err[i] * k_t[j];
        float ret = 1.0f - alpha[t];
        for (int64_t i = 0; i < dd; i++) m_n[i] = ret * m_t[i] + s_n[i];
        clamp_m_norm(m_n, dd, m_norm_max);
        for (int i = 0; i < d; i++) {
            float s = 0.0f;
            for (int j = 0; j < d; j++) s += m_n[i * d + j] * q_t[j];
            y[(int64_t)t * d + i] = s;
        }
    }
}

ORC_API void orc_titans_backward(const float* k_mem, const float* v_mem, const float* q_mem,
                                 const float* alpha, const float* theta, const float* eta,
                                 const float* m_states, const float* s_states, const float* d_y,
                                 const float* d_m_seed, const float* d_s_seed,
                                 float* d_k, float* d_v, float* d_q,
                                 float* d_alpha, float* d_theta, float* d_eta,
                                 float* d_m_out, float* d_s_out,
                                 int seq_len, int d, float error_clip) {
    const int64_t dd = (int64_t)d * d;
    std::vector<float> dM(dd, 0.0f), dS(dd, 0.0f), dMp(dd), pred(d), err(d), derr(d);
    if (d_m_seed) std::memcpy(dM.data(), d_m_seed, dd * sizeof(float));
    if (d_s_seed) std::memcpy(dS.data(), d_s_seed, dd * sizeof(float));
    for (int t = seq_len - 1; t >= 0; t--) {
        const float* k_t = k_mem + (int64_t)t * d;
        const float* v_t = v_mem + (int64_t)t * d;
        const float* q_t = q_mem + (int64_t)t * d;
        const float* dy = d_y + (int64_t)t * d;
        const float* m_t = m_states + (int64_t)t * dd;
        const float* m_n = m_states + (int64_t)(t + 1) * dd;
        const float* s_t = s_states + (int64_t)t * dd;
        float th = theta[t], et = eta[t];
        for (int i = 0; i < d; i++)
            for (int j = 0; j < d; j++) dM[i * d + j] += dy[i] * q_t[j];
        for (int j = 0; j < d; j++) {
            float s = 0.0f;
            for (int i = 0; i < d; i++) s += m_n[i * d + j] * dy[i];
            d_q[(int64_t)t * d + j] = s;
        }
        for (int64_t i = 0; i < dd; i++) dS[i] += dM[i];
        float da = 0.0f;
        for (int64_t i = 0; i < dd; i++) da += m_t[i] * dM[i];
        d_alpha[t] = -da;
        float ret = 1.0f - alpha[t];
        for (int64_t i = 0; i < dd; i++) dMp[i] = ret * dM[i];
        float de = 0.0f;
        for (int64_t i = 0; i < dd; i++) de += s_t[i] * dS[i];
        d_eta[t] = de;
        for (int i = 0; i < d; i++) {
            float s = 0.0f;
            for (int j = 0; j < d; j++) s += m_t[i * d + j] * k_t[j];
            pred[i] = s;
        }
        for (int i = 0; i < d; i++) err[i] = pred[i] - v_t[i];
        clip_error_l2(err.data(), d, error_clip);
        float dt = 0.0f;
        for (int i = 0; i < d; i++)
            for (int j = 0; j < d; j++) dt += err[i] * k_t[j] * dS[i * d + j];
        d_theta[t] = -dt;
        for (int i = 0; i < d; i++) {
            float s = 0.0f;
            for (int j = 0; j < d; j++) s += (-th * dS[i * d + j]) * k_t[j];
            derr[i] = s;
        }
        for (int j = 0; j < d; j++) {
            float s = 0.0f;
            for (int i = 0; i < d; i++) s += (-th * dS[i * d + j]) * err[i];
            d_k[(int64_t)t * d + j] = s;
        }
        for (int j = 0; j < d; j++) {
            float s = 0.0f;
            for (int i = 0; i < d; i++) s += m_t[i * d + j] * derr[i];
            d_k[(int64_t)t * d + j] += s;
        }
        for (int i = 0; i < d; i++) d_v[(int64_t)t * d + i] = -derr[i];
        for (int64_t i = 0; i < dd; i++) dS[i] = et * dS[i];
        for (int i = 0; i < d; i++)
            for (int j = 0; j < d; j++) dMp[i * d + j] += derr[i] * k_t[j];
        dM.swap(dMp);
    }
    std::memcpy(d_m_out, dM.data(), dd * sizeof(float));
    std::memcpy(d_s_out, dS.data(), dd * sizeof(float));
}

// ───────────────────────── Hebbian (core/src/dispatch.rs:1566-1660) ───────
ORC_API void orc_hebbian_forward(const float* k_mem, const float* v_mem, const float* q_mem,
                                 const float* alpha, const float* m_initial,
                                 float* m_states, float* y, int seq_len, int d, float m_norm_max) {
    const int64_t dd = (int64_t)d * d;
    std::memcpy(m_states, m_initial, dd * sizeof(float));
    for (int t = 0; t < seq_len; t++) {
        const float* k_t = k_mem + (int64_t)t * d;
        const float* v_t = v_mem + (int64_t)t * d;
        const float* q_t = q_mem + (int64_t)t * d;
        const float* m_t = m_states + (int64_t)t * dd;
        float* m_n = m_states + (int64_t)(t + 1) * dd;
        float ret = 1.0f - alpha[t];
        for (int i = 0; i < d; i++)
            for (int j = 0; j < d; j++)
                m_n[i * d + j] = ret * m_t[i * d + j] + v_t[i] * k_t[j];
        clamp_m_norm(m_n, dd, m_norm_max);
        for (int i = 0; i < d; i++) {
            float s = 0.0f;
            for (int j = 0; j < d; j++) s += m_n[i * d + j] * q_t[j];
            y[(int64_t)t * d + i] = s;
        }
    }
}

ORC_API void orc_hebbian_backward(const float* k_mem, const float* v_mem, const float* q_mem,
                                  const float* alpha, const float* m_states, const float* d_y,
                                  const float* d_m_seed,
                                  float* d_k, float* d_v, float* d_q, float* d_alpha,
                                  float* d_m_out, int seq_len, int d) {
    const int64_t dd = (int64_t)d * d;
    std::vector<float> dM(dd, 0.0f);
    if (d_m_seed) std::memcpy(dM.data(), d_m_seed, dd * sizeof(float));
    for (int t = seq_len - 1; t >= 0; t--) {
        const float* k_t = k_mem + (int64_t)t * d;
        const float* v_t = v_mem + (int64_t)t * d;
        const float* q_t = q_mem + (int64_t)t * d;
        const float* dy = d_y + (int64_t)t * d;
        const float* m_t = m_states + (int64_t)t * dd;
        const float* m_n = m_states + (int64_t)(t + 1) * dd;
        for (int i = 0; i < d; i++)
            for (int j = 0; j < d; j++) dM[i * d + j] += dy[i] * q_t[j];
        for (int j = 0; j < d; j++) {
            float s = 0.0f;
            for (int i = 0; i < d; i++) s += m_n[i * d + j] * dy[i];
            d_q[(int64_t)t * d + j] = s;
        }
        float da = 0.0f;
        for (int64_t i = 0; i < dd; i++) da += m_t[i] * dM[i];
        d_alpha[t] = -da;
        for (int i = 0; i < d; i++) {
            float s = 0.0f;
            for (int j = 0; j < d; j++) s += dM[i * d + j] * k_t[j];
            d_v[(int64_t)t * d + i] = s;
        }
        for (int j = 0; j < d; j++) {
            float s = 0.0f;
            for (int i = 0; i < d; i++) s += dM[i * d + j] * v_t[i];
            d_k[(int64_t)t * d + j] = s;
        }
        float ret = 1.0f - alpha[t];
        for (int64_t i = 0; i < dd; i++) dM[i] = ret * dM[i];
    }
    std::memcpy(d_m_out, dM.data(), dd * sizeof(float));
}

// ───────────────────────── frozen-M0 chunkwise ────────────────────────────
// The reference has no Rust statement of this recurrence; these follow the
// CUDA sources: core/kernels/titans_chunkwise_forward.cu:89-176,
// titans_chunkwise_backward.cu:118-358, delta_chunkwise_forward.cu:85-170,
// delta_chunkwise_backward.cu:118-330. `has_s` = 1 Titans, 0 Delta.
// m_norm projection uses the CUDA disable rule (<=0 or >=1e30 → off).
static void project_m_cuda(float* m, int64_t dd, float m_norm_max) {
    if (m_norm_max <= 0.0f || m_norm_max >= 1e30f) return;
    float nsq = 0.0f;
    for (int64_t i = 0; i < dd; i++) nsq += m[i] * m[i];
    float n = std::sqrt(nsq);
    if (n > m_norm_max) {
        float s = m_norm_max / n;
        for (int64_t i = 0; i < dd; i++) m[i] *= s;
    }
}

ORC_API void orc_chunkwise_forward(int has_s,
                                   const float* k_mem, const float* v_mem, const float* q_mem,
                                   const float* alpha, const float* theta, const float* eta,
                                   const float* m_initial, const float* s_initial,
                                   float* m_chunk_states, float* s_chunk_states, float* y,
                                   int seq_len, int d, int chunk_size,
                                   float error_clip, float m_norm_max) {
    const int64_t dd = (int64_t)d * d;
    const int num_chunks = (seq_len + chunk_size - 1) / chunk_size;
    std::vector<float> M(m_initial, m_initial + dd), S(dd, 0.0f);
    if (has_s) std::memcpy(S.data(), s_initial, dd * sizeof(float));
    std::vector<float> errs((size_t)chunk_size * d);
    for (int c = 0; c < num_chunks; c++) {
        int t0 = c * chunk_size;
        int t1 = std::min(t0 + chunk_size, seq_len);
        int C = t1 - t0;
        std::memcpy(m_chunk_states + (int64_t)c * dd, M.data(), dd * sizeof(float));
        if (has_s) std::memcpy(s_chunk_states + (int64_t)c * dd, S.data(), dd * sizeof(float));
        for (int tl = 0; tl < C; tl++) {  // phase 1: errors against frozen M0
            const float* k_t = k_mem + (int64_t)(t0 + tl) * d;
            const float* v_t = v_mem + (int64_t)(t0 + tl) * d;
            float* e = errs.data() + (size_t)tl * d;
            for (int i = 0; i < d; i++) {
                float s = 0.0f;
                for (int j = 0; j < d; j++) s += M[i * d + j] * k_t[j];
                e[i] = s - v_t[i];
            }
            clip_error_l2(e, d, error_clip);
        }
        for (int tl = 0; tl < C; tl++) {  // phase 2: sequential recurrence
            int t = t0 + tl;
            const float* k_t = k_mem + (int64_t)t * d;
            const float* q_t = q_mem + (int64_t)t * d;
            const float* e = errs.data() + (size_t)tl * d;
            float ret = 1.0f - alpha[t], th = theta[t];
            if (has_s) {
                float et = eta[t];
                for (int i = 0; i < d; i++)
                    for (int j = 0; j < d; j++) {
                        float sn = et * S[i * d + j] - th * e[i] * k_t[j];
                        S[i * d + j] = sn;
                        M[i * d + j] = ret * M[i * d + j] + sn;
                    }
            } else {
                for (int i = 0; i < d; i++)
                    for (int j = 0; j < d; j++)
                        M[i * d + j] = ret * M[i * d + j] - th * e[i] * k_t[j];
            }
            project_m_cuda(M.data(), dd, m_norm_max);
            for (int i = 0; i < d; i++) {
                float s = 0.0f;
                for (int j = 0; j < d; j++) s += M[i * d + j] * q_t[j];
                y[(int64_t)t * d + i] = s;
            }
        }
    }
    std::memcpy(m_chunk_states + (int64_t)num_chunks * dd, M.data(), dd * sizeof(float));
    if (has_s) std::memcpy(s_chunk_states + (int64_t)num_chunks * dd, S.data(), dd * sizeof(float));
}

ORC_API void orc_chunkwise_backward(int has_s,
                                    const float* k_mem, const float* v_mem, const float* q_mem,
                                    const float* alpha, const float* theta, const float* eta,
                                    const float* m_chunk_states, const float* s_chunk_states,
                                    const float* d_y,
                                    float* d_k, float* d_v, float* d_q,
                                    float* d_alpha, float* d_theta, float* d_eta,
                                    float* d_m_out, float* d_s_out,
                                    int seq_len, int d, int chunk_size,
                                    float error_clip, float m_norm_max) {
    const int64_t dd = (int64_t)d * d;
    const int num_chunks = (seq_len + chunk_size - 1) / chunk_size;
    std::vector<float> dM(dd, 0.0f), dS(dd, 0.0f), dM0(dd);
    std::vector<float> mrec((size_t)(chunk_size + 1) * dd), srec;
    if (has_s) srec.resize((size_t)(chunk_size + 1) * dd);
    std::vector<float> errs((size_t)chunk_size * d), derr(d);
    for (int c = num_chunks - 1; c >= 0; c--) {
        int t0 = c * chunk_size;
        int t1 = std::min(t0 + chunk_size, seq_len);
        int C = t1 - t0;
        std::memcpy(mrec.data(), m_chunk_states + (int64_t)c * dd, dd * sizeof(float));
        if (has_s) std::memcpy(srec.data(), s_chunk_states + (int64_t)c * dd, dd * sizeof(float));
        const float* M0 = mrec.data();
        for (int tl = 0; tl < C; tl++) {
            const float* k_t = k_mem + (int64_t)(t0 + tl) * d;
            const float* v_t = v_mem + (int64_t)(t0 + tl) * d;
            float* e = errs.data() + (size_t)tl * d;
            for (int i = 0; i < d; i++) {
                float s = 0.0f;
                for (int j = 0; j < d; j++) s += M0[i * d + j] * k_t[j];
                e[i] = s - v_t[i];
            }
            clip_error_l2(e, d, error_clip);
        }
        for (int tl = 0; tl < C; tl++) {
            int t = t0 + tl;
            const float* k_t = k_mem + (int64_t)t * d;
            const float* e = errs.data() + (size_t)tl * d;
            const float* mc = mrec.data() + (size_t)tl * dd;
            float* mn = mrec.data() + (size_t)(tl + 1) * dd;
            float ret = 1.0f - alpha[t], th = theta[t];
            if (has_s) {
                const float* sc = srec.data() + (size_t)tl * dd;
                float* sn = srec.data() + (size_t)(tl + 1) * dd;
                float et = eta[t];
                for (int i = 0; i < d; i++)
                    for (int j = 0; j < d; j++) {
                        float v = et * sc[i * d + j] - th * e[i] * k_t[j];
                        sn[i * d + j] = v;
                        mn[i * d + j] = ret * mc[i * d + j] + v;
                    }
            } else {
                for (int i = 0; i < d; i++)
                    for (int j = 0; j < d; j++)
                        mn[i * d + j] = ret * mc[i * d + j] - th * e[i] * k_t[j];
            }
            project_m_cuda(mn, dd, m_norm_max);
        }
        std::fill(dM0.begin(), dM0.end(), 0.0f);
        for (int tl = C - 1; tl >= 0; tl--) {
            int t = t0 + tl;
            const float* k_t = k_mem + (int64_t)t * d;
            const float* q_t = q_mem + (int64_t)t * d;
            const float* dy = d_y + (int64_t)t * d;
            const float* m_t = mrec.data() + (size_t)tl * dd;
            const float* m_n = mrec.data() + (size_t)(tl + 1) * dd;
            const float* e = errs.data() + (size_t)tl * d;
            float th = theta[t], ret = 1.0f - alpha[t];
            for (int i = 0; i < d; i++)
                for (int j = 0; j < d; j++) dM[i * d + j] += dy[i] * q_t[j];
            for (int j = 0; j < d; j++) {
                float s = 0.0f;
                for (int i = 0; i < d; i++) s += m_n[i * d + j] * dy[i];
                d_q[(int64_t)t * d + j] = s;
            }
            if (has_s) for (int64_t i = 0; i < dd; i++) dS[i] += dM[i];
            float da = 0.0f;
            for (int64_t i = 0; i < dd; i++) da += m_t[i] * dM[i];
            d_alpha[t] = -da;
            float* G;  // gradient that multiplies the outer(e,k) term
            if (has_s) {
                for (int64_t i = 0; i < dd; i++) dM[i] = ret * dM[i];
                const float* s_t = srec.data() + (size_t)tl * dd;
                float de = 0.0f;
                for (int64_t i = 0; i < dd; i++) de += s_t[i] * dS[i];
                d_eta[t] = de;
                G = dS.data();
            } else {
                G = dM.data();  // Delta: uses d_M before the retention scaling
            }
            float dt = 0.0f;
            for (int i = 0; i < d; i++)
                for (int j = 0; j < d; j++) dt += e[i] * k_t[j] * G[i * d + j];
            d_theta[t] = -dt;
            for (int i = 0; i < d; i++) {
                float s = 0.0f;
                for (int j = 0; j < d; j++) s += (-th * G[i * d + j]) * k_t[j];
                derr[i] = s;
            }
            for (int j = 0; j < d; j++) {
                float s = 0.0f;
                for (int i = 0; i < d; i++) s += (-th * G[i * d + j]) * e[i];
                d_k[(int64_t)t * d + j] = s;
            }
            for (int j = 0; j < d; j++) {
                float s = 0.0f;
                for (int i = 0; i < d; i++) s += M0[i * d + j] * derr[i];
                d_k[(int64_t)t * d + j] += s;
            }
            for (int i = 0; i < d; i++) d_v[(int64_t)t * d + i] = -derr[i];
            if (has_s) {
                float et = eta[t];
                for (int64_t i = 0; i < dd; i++) dS[i] = et * dS[i];
            } else {
                for (int64_t i = 0; i < dd; i++) dM[i] = ret * dM[i];
            }
            for (int i = 0; i < d; i++)
                for (int j = 0; j < d; j++) dM0[i * d + j] += derr[i] * k_t[j];
        }
        for (int64_t i = 0; i < dd; i++) dM[i] += dM0[i];
    }
    std::memcpy(d_m_out, dM.data(), dd * sizeof(float));
    if (has_s) std::memcpy(d_s_out, dS.data(), dd * sizeof(float));
}

// ───────────────────────── SWA (core/src/swa.rs:33-92, 163-235) ───────────
// Layout: q,k,v,out [seq, nh*hd]; attn_weights [nh, seq, n_persistent+window].
// The persistent-prefix mask (n_persistent > 0) follows the CUDA kernel
// core/kernels/swa_forward.cu:48-60: slots [0,n_p) hold keys 0..n_p-1 (those
// <= q_pos), slots n_p+w hold keys local_start+w. n_persistent = 0 is exactly
// the Rust reference.
static inline void swa_ranges(int q_pos, int window, int n_p, int* n_p_attend,
                              int* local_start, int* local_len) {
    *n_p_attend = (q_pos + 1 < n_p) ? (q_pos + 1) : n_p;
    if (q_pos >= n_p) {
        int ls = (q_pos + 1 - window > n_p) ? (q_pos + 1 - window) : n_p;
        *local_start = ls;
        *local_len = q_pos + 1 - ls;
    } else {
        *local_start = 0;
        *local_len = 0;
    }
}

ORC_API void orc_swa_forward(const float* q, const float* k, const float* v,
                             float* out, float* attn_weights,
                             int seq_len, int num_heads, int head_dim, int window, int n_p) {
    const int td = num_heads * head_dim;
    const int aw = n_p + window;
    const float scale = 1.0f / std::sqrt((float)head_dim);
    std::fill(out, out + (int64_t)seq_len * td, 0.0f);
    std::fill(attn_weights, attn_weights + (int64_t)num_heads * seq_len * aw, 0.0f);
    std::vector<float> scores(aw);
    const float NEG = -std::numeric_limits<float>::infinity();
    for (int h = 0; h < num_heads; h++) {
        int ho = h * head_dim;
        for (int qp = 0; qp < seq_len; qp++) {
            int npa, ls, ll;
            swa_ranges(qp, window, n_p, &npa, &ls, &ll);
            std::fill(scores.begin(), scores.end(), NEG);
            for (int w = 0; w < npa; w++) {
                float dot = 0.0f;
                for (int dd = 0; dd < head_dim; dd++)
                    dot += q[(int64_t)qp * td + ho + dd] * k[(int64_t)w * td + ho + dd];
                scores[w] = dot * scale;
            }
            for (int w = 0; w < ll; w++) {
                int kp = ls + w;
                float dot = 0.0f;
                for (int dd = 0; dd < head_dim; dd++)
                    dot += q[(int64_t)qp * td + ho + dd] * k[(int64_t)kp * td + ho + dd];
                scores[n_p + w] = dot * scale;
            }
            // softmax_f32 (core/src/tensor.rs softmax: max-subtract, exp, normalise)
            float mx = NEG;
            for (int w = 0; w < aw; w++) mx = std::max(mx, scores[w]);
            float* wrow = attn_weights + ((int64_t)h * seq_len + qp) * aw;
            float sum = 0.0f;
            for (int w = 0; w < aw; w++) {
                float e = std::exp(scores[w] - mx);
                wrow[w] = e;
                sum += e;
            }
            for (int w = 0; w < aw; w++) wrow[w] /= sum;
            for (int w = 0; w < npa; w++) {
                float wt = wrow[w];
                for (int dd = 0; dd < head_dim; dd++)
                    out[(int64_t)qp * td + ho + dd] += wt * v[(int64_t)w * td + ho + dd];
            }
            for (int w = 0; w < ll; w++) {
                int kp = ls + w;
                float wt = wrow[n_p + w];
                for (int dd = 0; dd < head_dim; dd++)
                    out[(int64_t)qp * td + ho + dd] += wt * v[(int64_t)kp * td + ho + dd];
            }
        }
    }
}

// d_q,d_k,d_v are accumulated into (caller zeroes), as in swa_backward_rust.
ORC_API void orc_swa_backward(const float* q, const float* k, const float* v,
                              const float* attn_weights, const float* d_out,
                              float* d_q, float* d_k, float* d_v,
                              int seq_len, int num_heads, int head_dim, int window, int n_p) {
    const int td = num_heads * head_dim;
    const int aw = n_p + window;
    const float scale = 1.0f / std::sqrt((float)head_dim);
    std::vector<float> daw(aw), dsc(aw);
    std::vector<int> kpos(aw);
    for (int h = 0; h < num_heads; h++) {
        int ho = h * head_dim;
        for (int qp = 0; qp < seq_len; qp++) {
            int npa, ls, ll;
            swa_ranges(qp, window, n_p, &npa, &ls, &ll);
            const float* wrow = attn_weights + ((int64_t)h * seq_len + qp) * aw;
            // valid slots in order: persistent then local
            int nv = 0;
            std::vector<int>& kp = kpos;
            std::vector<int> slot(aw);
            for (int w = 0; w < npa; w++) { kp[nv] = w; slot[nv] = w; nv++; }
            for (int w = 0; w < ll; w++) { kp[nv] = ls + w; slot[nv] = n_p + w; nv++; }
            for (int i = 0; i < nv; i++) {
                float s = 0.0f;
                for (int dd = 0; dd < head_dim; dd++)
                    s += d_out[(int64_t)qp * td + ho + dd] * v[(int64_t)kp[i] * td + ho + dd];
                daw[i] = s;
            }
            for (int i = 0; i < nv; i++) {
                float a = wrow[slot[i]];
                for (int dd = 0; dd < head_dim; dd++)
                    d_v[(int64_t)kp[i] * td + ho + dd] += a * d_out[(int64_t)qp * td + ho + dd];
            }
            float dot = 0.0f;
            for (int i = 0; i < nv; i++) dot += wrow[slot[i]] * daw[i];
            for (int i = 0; i < nv; i++) dsc[i] = wrow[slot[i]] * (daw[i] - dot);
            for (int i = 0; i < nv; i++) {
                float ds = dsc[i] * scale;
                for (int dd = 0; dd < head_dim; dd++) {
                    d_q[(int64_t)qp * td + ho + dd] += ds * k[(int64_t)kp[i] * td + ho + dd];
                    d_k[(int64_t)kp[i] * td + ho + dd] += ds * q[(int64_t)qp * td + ho + dd];
                }
            }
        }
    }
}

// ───────────────────────── AdamW (core/src/adamw.rs:102-124) ──────────────
ORC_API void orc_adamw_step(float* w, const float* g, float* m, float* v, int64_t n,
                            float lr, float beta1, float beta2, float eps,
                            float bc1_inv, float bc2_inv, float weight_decay) {
    for (int64_t i = 0; i < n; i++) {
        float gi = g[i];
        m[i] = beta1 * m[i] + (1.0f - beta1) * gi;
        v[i] = beta2 * v[i] + (1.0f - beta2) * gi * gi;
        float mh = m[i] * bc1_inv;
        float vh = v[i] * bc2_inv;
        w[i] -= lr * (mh / (std::sqrt(vh) + eps) + weight_decay * w[i]);
    }
}

// Global-norm clip (core/kernels/adamw.cu:205-236; gpu_stacked_optimizer.rs:193-345):
// norm = sqrt(sum g^2); scale = max_norm/norm if norm > max_norm > 0 else 1.
ORC_API float orc_grad_norm_clip(float* g, int64_t n, float max_norm, float* out_scale) {
    double acc = 0.0;  // partial sums in the reference are f32 per 256 block; f64 here is the tighter truth
    for (int64_t i = 0; i < n; i++) acc += (double)g[i] * (double)g[i];
    float norm = (float)std::sqrt(acc);
    float scale = (norm > max_norm && max_norm > 0.0f) ? (max_norm / norm) : 1.0f;
    if (out_scale) *out_scale = scale;
    if (scale < 1.0f) for (int64_t i = 0; i < n; i++) g[i] *= scale;
    return norm;
}

// ───────────────────────── gates (rule wrapper pre-step) ──────────────────
// alpha = clamp(sigmoid(c·w_a + b_a)), theta = clamp(softplus(c·w_t + b_t)),
// eta = sigmoid(c·w_e + b_e), c = [k_hat ; v] (core/src/titans_lmm.rs:1423-1445).
// which: 0 sigmoid, 1 softplus. Returns pre-activation in pre[], value in out[].
ORC_API void orc_gate(const float* k, const float* v, const float* w, float b, int which,
                      float lo, float hi, int has_clamp, float* pre, float* out,
                      int64_t n_tok, int d) {
    for (int64_t t = 0; t < n_tok; t++) {
        float s = b;
        for (int j = 0; j < d; j++) s += k[t * d + j] * w[j];
        for (int j = 0; j < d; j++) s += v[t * d + j] * w[d + j];
        pre[t] = s;
        float a = which == 0 ? sigmoid_f32(s) : softplus_f32(s);
        if (has_clamp) a = std::min(std::max(a, lo), hi);
        out[t] = a;
    }
}

// ───────────────────────── batched / threaded drivers (CPU baseline) ──────
template <class F>
static void run_mt(int n_items, int n_threads, F fn) {
    if (n_threads <= 1) { for (int i = 0; i < n_items; i++) fn(i); return; }
    std::vector<std::thread> th;
    for (int w = 0; w < n_threads; w++)
        th.emplace_back([=]() { for (int i = w; i < n_items; i += n_threads) fn(i); });
    for (auto& t : th) t.join();
}

// Titans exact fwd+bwd over `batch` independent problems ([N,S,d] layout).
// Per-problem d_m/d_s outputs: d_m_out [N,dd].
ORC_API void orc_titans_fwd_bwd_batched_mt(
    const float* k, const float* v, const float* q, const float* alpha, const float* theta,
    const float* eta, const float* m0, const float* s0, const float* d_y,
    float* m_states, float* s_states, float* y,
    float* d_k, float* d_v, float* d_q, float* d_alpha, float* d_theta, float* d_eta,
    float* d_m_out, float* d_s_out,
    int batch, int seq_len, int d, float error_clip, float m_norm_max, int n_threads) {
    const int64_t dd = (int64_t)d * d, sd = (int64_t)seq_len * d, tr = (int64_t)(seq_len + 1) * dd;
    run_mt(batch, n_threads, [=](int b) {
        orc_titans_forward(k + b * sd, v + b * sd, q + b * sd, alpha + (int64_t)b * seq_len,
                           theta + (int64_t)b * seq_len, eta + (int64_t)b * seq_len,
                           m0 + b * dd, s0 + b * dd, m_states + b * tr, s_states + b * tr,
                           y + b * sd, seq_len, d, error_clip, m_norm_max);
        orc_titans_backward(k + b * sd, v + b * sd, q + b * sd, alpha + (int64_t)b * seq_len,
                            theta + (int64_t)b * seq_len, eta + (int64_t)b * seq_len,
                            m_states + b * tr, s_states + b * tr, d_y + b * sd, nullptr, nullptr,
                            d_k + b * sd, d_v + b * sd, d_q + b * sd,
                            d_alpha + (int64_t)b * seq_len, d_theta + (int64_t)b * seq_len,
                            d_eta + (int64_t)b * seq_len, d_m_out + b * dd, d_s_out + b * dd,
                            seq_len, d, error_clip);
    });
}

ORC_API void orc_chunkwise_fwd_bwd_batched_mt(
    int has_s, const float* k, const float* v, const float* q, const float* alpha,
    const float* theta, const float* eta, const float* m0, const float* s0, const float* d_y,
    float* m_chunk, float* s_chunk, float* y,
    float* d_k, float* d_v, float* d_q, float* d_alpha, float* d_theta, float* d_eta,
    float* d_m_out, float* d_s_out,
    int batch, int seq_len, int d, int chunk, float error_clip, float m_norm_max, int n_threads) {
    const int64_t dd = (int64_t)d * d, sd = (int64_t)seq_len * d;
    const int nc = (seq_len + chunk - 1) / chunk;
    const int64_t cs = (int64_t)(nc + 1) * dd;
    run_mt(batch, n_threads, [=](int b) {
        const int64_t so = (int64_t)b * seq_len;
        orc_chunkwise_forward(has_s, k + b * sd, v + b * sd, q + b * sd, alpha + so, theta + so,
                              has_s ? eta + so : nullptr, m0 + b * dd, has_s ? s0 + b * dd : nullptr,
                              m_chunk + b * cs, has_s ? s_chunk + b * cs : nullptr, y + b * sd,
                              seq_len, d, chunk, error_clip, m_norm_max);
        orc_chunkwise_backward(has_s, k + b * sd, v + b * sd, q + b * sd, alpha + so, theta + so,
                               has_s ? eta + so : nullptr, m_chunk + b * cs,
                               has_s ? s_chunk + b * cs : nullptr, d_y + b * sd,
                               d_k + b * sd, d_v + b * sd, d_q + b * sd, d_alpha + so, d_theta + so,
                               has_s ? d_eta + so : nullptr, d_m_out + b * dd,
                               has_s ? d_s_out + b * dd : nullptr,
                               seq_len, d, chunk, error_clip, m_norm_max);
    });
}

// SWA fwd+bwd over `batch` independent sequences, threads over (batch).
ORC_API void orc_swa_fwd_bwd_batched_mt(
    const float* q, const float* k, const float* v, const float* d_out,
    float* out, float* attn_w, float* d_q, float* d_k, float* d_v,
    int batch, int seq_len, int num_heads, int head_dim, int window, int n_p, int n_threads) {
    const int64_t sz = (int64_t)seq_len * num_heads * head_dim;
    const int64_t awz = (int64_t)num_heads * seq_len * (n_p + window);
    run_mt(batch, n_threads, [=](int b) {
        orc_swa_forward(q + b * sz, k + b * sz, v + b * sz, out + b * sz, attn_w + b * awz,
                        seq_len, num_heads, head_dim, window, n_p);
        orc_swa_backward(q + b * sz, k + b * sz, v + b * sz, attn_w + b * awz, d_out + b * sz,
                         d_q + b * sz, d_k + b * sz, d_v + b * sz,
                         seq_len, num_heads, head_dim, window, n_p);
    });
}

ORC_API void orc_adamw_step_mt(float* w, const float* g, float* m, float* v, int64_t n,
                               float lr, float beta1, float beta2, float eps,
                               float bc1_inv, float bc2_inv, float wd, int n_threads) {
    int64_t per = (n + n_threads - 1) / n_threads;
    run_mt(n_threads, n_threads, [=](int i) {
        int64_t a = (int64_t)i * per, b = std::min(n, a + per);
        if (a < b) orc_adamw_step(w + a, g + a, m + a, v + a, b - a, lr, beta1, beta2, eps,
                                  bc1_inv, bc2_inv, wd);
    });
}

ORC_API int orc_hardware_threads() {
    unsigned n = std::thread::hardware_concurrency();
    return n == 0 ? 1 : (int)n;
}
