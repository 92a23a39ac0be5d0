// Shared host/device helpers for the NL_Hecate B200 kernel library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

// ── status codes returned by the status-returning entry points ────────────
#define NLH_OK 0
#define NLH_ERR_INVALID_ARG 1
#define NLH_ERR_CUDA 2
#define NLH_ERR_WORKSPACE 3
#define NLH_ERR_TIMEOUT 4
#define NLH_ERR_UNSUPPORTED 5

namespace nlh {

// Stream every launch of the library goes to. Defaults to the legacy default
// stream, which is what the reference's wrappers use (no stream argument in
// core/src/cuda_ffi.rs). Set with nlh_set_stream().
cudaStream_t current_stream();

// Last non-OK status recorded by a void entry point (the reference aborts the
// process instead: core/kernels/titans_forward.cu:67-81).
void record_status(int status, const char* where, const char* detail);

// Value of a library option (nlh_set_option); unknown options read 0.
int option_value(int option);

// Grow-only per-device scratch. Returned pointer is 256-byte aligned and is
// valid until the next call that asks for more bytes on the same device.
// Returns nullptr (and records NLH_ERR_WORKSPACE) on failure.
void* workspace(size_t bytes);

inline bool check_launch(const char* where) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        record_status(NLH_ERR_CUDA, where, cudaGetErrorString(e));
        return false;
    }
    return true;
}

enum Rule { RULE_DELTA = 0, RULE_TITANS = 1, RULE_HEBBIAN = 2 };

// How the forward kernels emit memory states.
enum StoreMode {
    STORE_ALL = 0,    // slot 0 = initial, slot t+1 after every token   [(S+1) slots]
    STORE_CKPT = 1,   // slot 0 = initial, then every `interval` tokens and the final state
    STORE_CHUNK = 2,  // slot c = state at the start of chunk c, slot num_chunks = final
    STORE_FINAL = 3   // slot 0 = final state only
};

struct FwdArgs {
    const float *k, *v, *q, *alpha, *theta, *eta;
    const float *m_init, *s_init;
    float *m_out, *s_out, *y;
    float *m_work, *s_work;    // [batch, d*d] (unused in STORE_ALL)
    int seq_len, d, batch;
    long long in_stride_tok;   // tokens between batch elements of k/v/q/gates
    long long init_stride;     // floats between batch elements of m_init/s_init
    long long out_stride;      // floats between batch elements of m_out/s_out
    int store_mode, interval;  // interval: checkpoint interval or chunk size
    int frozen;                // errors are taken against the chunk-start state
    float error_clip, m_norm_max;
};

struct BwdArgs {
    const float *k, *v, *q, *alpha, *theta, *eta;
    const float *m_traj, *s_traj;  // STORE_ALL-style trajectory, or chunk-boundary states if frozen
    const float *d_y;
    const float *d_m_seed, *d_s_seed;  // nullable; [batch, d*d]
    float *d_k, *d_v, *d_q, *d_alpha, *d_theta, *d_eta;
    float *d_m_out, *d_s_out;
    float *dM, *dS, *dM0;          // work [batch, d*d]
    float *m_rec, *s_rec;          // frozen: recomputed chunk trajectory [batch, (chunk+1)*d*d]
    int seq_len, d, batch;         // seq_len = tokens between batch elements of the streams
    int t_start, t_end;            // token range processed (reverse)
    long long traj_stride;         // floats between batch elements of m_traj/s_traj
    int frozen, chunk;
    int atomic_out;                // 1: atomicAdd into one shared [d*d]; 0: store per batch element
    float error_clip, m_norm_max;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over the whole block; every thread gets the same (deterministic) total.
// red must hold at least 32 floats. Contains two __syncthreads().
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nwarps; w++) t += red[w];
    __syncthreads();
    return t;
}

// Division of a non-negative 31-bit integer by a divisor fixed at launch: a shift for powers of
// two, otherwise one multiply-high and a shift (mul = ceil(2^(32+shr) / d), shr = floor(log2 d),
// exact for every n < 2^31). Replaces the ~20-instruction integer division in index arithmetic.
struct FastDiv {
    unsigned mul;
    int shr;
    int d;
};
inline FastDiv make_fastdiv(int d)
{
    FastDiv f;
    f.d = d < 1 ? 1 : d;
    int lg = 0;
    while ((1LL << (lg + 1)) <= f.d) lg++;
    f.shr = lg;
    if ((1LL << lg) == f.d) { f.mul = 0; return f; }
    const unsigned long long num = 1ULL << (32 + lg);
    f.mul = (unsigned)((num + (unsigned long long)f.d - 1) / (unsigned long long)f.d);
    return f;
}
__device__ __forceinline__ int fd_div(int n, const FastDiv& f)
{
    return f.mul ? (int)(__umulhi((unsigned)n, f.mul) >> f.shr) : (n >> f.shr);
}

__host__ __device__ __forceinline__ bool m_norm_enabled(float m_norm_max) {
    // core/kernels/m_norm_project.cuh: disabled when <= 0 or >= 1e30.
    return m_norm_max > 0.0f && m_norm_max < 1e30f;
}

}  // namespace nlh
