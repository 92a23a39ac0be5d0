// Sliding-window attention in fp32 end to end: the accuracy option of the SWA pair.
//
// The reference's CPU path (core/src/swa.rs:33-92 forward, :163-235 backward) is fp32 throughout;
// its GPU path and this library's tensor-core kernels take bf16 q, k, v. Configurations that are
// stated in fp32 (the reference's CPU-runnable model: d_model 64, one head, seq 256) run here, so
// that every output and gradient agrees with the fp32 reference to rounding (1e-4 relative)
// instead of to bf16 resolution. CUDA-core kernels, one warp per query (forward, dQ) or per key
// (dK, dV); cost O(S * window * head_dim) without tiling — meant for small fp32 shapes, not for
// the benchmark sizes (which use the tcgen05 kernels).
//
// Visible keys of query q: the persistent prefix [0, min(q+1, n_p)) and the local window
// [max(q+1-W, n_p), q] (core/kernels/swa_forward.cu:48-60 for the prefix rule).
#include "nlh_common.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {

constexpr int SF_WARPS = 4;
constexpr int SF_MAX_KEYS = 2048;     // n_persistent + window (scores of one query in shared memory)
constexpr int SF_CHUNK = 512;         // queries per pass of the dK/dV kernel

__device__ __forceinline__ bool sf_visible(int qp, int kp, int window, int n_p)
{
    return kp <= qp && (kp < n_p || kp >= qp + 1 - window);
}
// w-th visible key of query qp (prefix keys first, then the local window), or -1
__device__ __forceinline__ int sf_key(int w, int qp, int window, int n_p, int n_pre, int local_start)
{
    return (w < n_pre) ? w : local_start + (w - n_pre);
}

// grid: ceil(B*H*S / SF_WARPS); one warp per (b, h, query)
__global__ void __launch_bounds__(SF_WARPS * 32) swa_f32_fwd_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    float* __restrict__ out, float* __restrict__ lse, int S, int H, int hd, int window, int n_p, int B,
    float scale)
{
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* qs = sm + warp * (hd + SF_MAX_KEYS);
    float* sc = qs + hd;
    const long long row = (long long)blockIdx.x * SF_WARPS + warp;
    if (row >= (long long)B * H * S) return;
    const int qp = (int)(row % S), h = (int)((row / S) % H), b = (int)(row / ((long long)S * H));
    const size_t rs = (size_t)H * hd;
    const size_t base = (size_t)b * S * rs + (size_t)h * hd;
    for (int i = lane; i < hd; i += 32) qs[i] = q[base + (size_t)qp * rs + i];
    __syncwarp();
    const int n_pre = min(qp + 1, n_p);
    const int local_start = max(qp + 1 - window, n_p);
    const int n_loc = max(qp + 1 - local_start, 0);
    const int nk = n_pre + n_loc;
    float mx = -INFINITY;
    for (int w = lane; w < nk; w += 32) {
        const float* kr = k + base + (size_t)sf_key(w, qp, window, n_p, n_pre, local_start) * rs;
        float dot = 0.f;
        for (int i = 0; i < hd; i++) dot = fmaf(qs[i], kr[i], dot);
        const float s = dot * scale;
        sc[w] = s;
        mx = fmaxf(mx, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int w = lane; w < nk; w += 32) {
        const float p = expf(sc[w] - mx);
        sc[w] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    const float inv = sum > 0.f ? 1.0f / sum : 0.f;
    for (int i = lane; i < hd; i += 32) {
        float acc = 0.f;
        for (int w = 0; w < nk; w++)
            acc = fmaf(sc[w], v[base + (size_t)sf_key(w, qp, window, n_p, n_pre, local_start) * rs + i], acc);
        out[base + (size_t)qp * rs + i] = acc * inv;
    }
    if (lane == 0) lse[row] = mx + logf(sum);
}

// dQ: one warp per (b, h, query). delta = dO . O is formed here.
__global__ void __launch_bounds__(SF_WARPS * 32) swa_f32_dq_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ out, const float* __restrict__ lse, const float* __restrict__ d_out,
    float* __restrict__ d_q, int S, int H, int hd, int window, int n_p, int B, float scale)
{
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* qs = sm + warp * (2 * hd + SF_MAX_KEYS);
    float* gs = qs + hd;            // dO row
    float* sc = gs + hd;            // dS per visible key
    const long long row = (long long)blockIdx.x * SF_WARPS + warp;
    if (row >= (long long)B * H * S) return;
    const int qp = (int)(row % S), h = (int)((row / S) % H), b = (int)(row / ((long long)S * H));
    const size_t rs = (size_t)H * hd;
    const size_t base = (size_t)b * S * rs + (size_t)h * hd;
    float del = 0.f;
    for (int i = lane; i < hd; i += 32) {
        const size_t o = base + (size_t)qp * rs + i;
        qs[i] = q[o];
        gs[i] = d_out[o];
        del = fmaf(d_out[o], out[o], del);
    }
    del = warp_sum(del);
    __syncwarp();
    const float l = lse[row];
    const int n_pre = min(qp + 1, n_p);
    const int local_start = max(qp + 1 - window, n_p);
    const int nk = n_pre + max(qp + 1 - local_start, 0);
    for (int w = lane; w < nk; w += 32) {
        const size_t ko = base + (size_t)sf_key(w, qp, window, n_p, n_pre, local_start) * rs;
        float dot = 0.f, dp = 0.f;
        for (int i = 0; i < hd; i++) { dot = fmaf(qs[i], k[ko + i], dot); dp = fmaf(gs[i], v[ko + i], dp); }
        const float p = expf(dot * scale - l);
        sc[w] = p * (dp - del) * scale;
    }
    __syncwarp();
    for (int i = lane; i < hd; i += 32) {
        float acc = 0.f;
        for (int w = 0; w < nk; w++)
            acc = fmaf(sc[w], k[base + (size_t)sf_key(w, qp, window, n_p, n_pre, local_start) * rs + i], acc);
        d_q[base + (size_t)qp * rs + i] = acc;
    }
}

// dK, dV: one warp per (b, h, key); queries that see the key are walked in passes of SF_CHUNK.
template <bool ACCUM>
__global__ void __launch_bounds__(SF_WARPS * 32) swa_f32_dkv_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ out, const float* __restrict__ lse, const float* __restrict__ d_out,
    float* __restrict__ d_k, float* __restrict__ d_v, int S, int H, int hd, int window, int n_p, int B,
    float scale)
{
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* ks = sm + warp * (2 * hd + 2 * SF_CHUNK);
    float* vs = ks + hd;
    float* ps = vs + hd;            // P per query of the pass
    float* ds = ps + SF_CHUNK;      // dS per query of the pass
    const long long row = (long long)blockIdx.x * SF_WARPS + warp;
    if (row >= (long long)B * H * S) return;
    const int kp = (int)(row % S), h = (int)((row / S) % H), b = (int)(row / ((long long)S * H));
    const size_t rs = (size_t)H * hd;
    const size_t base = (size_t)b * S * rs + (size_t)h * hd;
    const float* lse_bh = lse + ((size_t)b * H + h) * S;
    for (int i = lane; i < hd; i += 32) { ks[i] = k[base + (size_t)kp * rs + i]; vs[i] = v[base + (size_t)kp * rs + i]; }
    __syncwarp();
    const int q_last = (kp < n_p) ? S - 1 : min(S - 1, kp + window - 1);
    // per-lane accumulators for dims i = lane + 32 j (head_dim <= 128)
    float akk[4] = {0.f, 0.f, 0.f, 0.f}, avv[4] = {0.f, 0.f, 0.f, 0.f};
    for (int q0 = kp; q0 <= q_last; q0 += SF_CHUNK) {
        const int nq = min(SF_CHUNK, q_last - q0 + 1);
        for (int w = lane; w < nq; w += 32) {
            const int qp = q0 + w;
            const size_t qo = base + (size_t)qp * rs;
            float dot = 0.f, dp = 0.f, del = 0.f;
            for (int i = 0; i < hd; i++) {
                const float g = d_out[qo + i];
                dot = fmaf(q[qo + i], ks[i], dot);
                dp = fmaf(g, vs[i], dp);
                del = fmaf(g, out[qo + i], del);
            }
            const float p = sf_visible(qp, kp, window, n_p) ? expf(dot * scale - lse_bh[qp]) : 0.f;
            ps[w] = p;
            ds[w] = p * (dp - del) * scale;
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i = lane + 32 * j;
            if (i < hd) {
                float a = akk[j], c = avv[j];
                for (int w = 0; w < nq; w++) {
                    const size_t qo = base + (size_t)(q0 + w) * rs + i;
                    a = fmaf(ds[w], q[qo], a);
                    c = fmaf(ps[w], d_out[qo], c);
                }
                akk[j] = a; avv[j] = c;
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int i = lane + 32 * j;
        if (i < hd) {
            const size_t o = base + (size_t)kp * rs + i;
            if (ACCUM) { d_k[o] += akk[j]; d_v[o] += avv[j]; }
            else { d_k[o] = akk[j]; d_v[o] = avv[j]; }
        }
    }
}

static int sf_check(const char* where, int S, int H, int hd, int W, int B, int n_p)
{
    if (S <= 0 || H <= 0 || hd <= 0 || B < 0 || W <= 0 || n_p < 0) {
        record_status(NLH_ERR_INVALID_ARG, where, "seq_len, num_heads, head_dim, window_size must be > 0; batch, n_persistent >= 0");
        return NLH_ERR_INVALID_ARG;
    }
    if (hd > 128 || n_p + (W < S ? W : S) > SF_MAX_KEYS) {
        record_status(NLH_ERR_UNSUPPORTED, where, "fp32 SWA: head_dim <= 128 and n_persistent + window <= 2048");
        return NLH_ERR_UNSUPPORTED;
    }
    return NLH_OK;
}

}  // namespace nlh

using namespace nlh;

extern "C" {

int32_t nlh_swa_forward_f32(const float* q, const float* k, const float* v, float* out, float* lse,
    int32_t seq_len, int32_t num_heads, int32_t head_dim, int32_t window_size, int32_t batch_size,
    int32_t n_persistent)
{
    int rc = sf_check("nlh_swa_forward_f32", seq_len, num_heads, head_dim, window_size, batch_size, n_persistent);
    if (rc != NLH_OK || batch_size == 0) return rc;
    if (!q || !k || !v || !out || !lse) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_swa_forward_f32", "NULL pointer");
        return NLH_ERR_INVALID_ARG;
    }
    const long long rows = (long long)batch_size * num_heads * seq_len;
    const size_t smem = (size_t)SF_WARPS * (head_dim + SF_MAX_KEYS) * sizeof(float);
    const int w = window_size < seq_len ? window_size : seq_len;
    swa_f32_fwd_kernel<<<(unsigned)((rows + SF_WARPS - 1) / SF_WARPS), SF_WARPS * 32, smem, current_stream()>>>(
        q, k, v, out, lse, seq_len, num_heads, head_dim, w, n_persistent, batch_size, 1.0f / sqrtf((float)head_dim));
    return check_launch("nlh_swa_forward_f32") ? NLH_OK : NLH_ERR_CUDA;
}

int32_t nlh_swa_backward_f32(const float* q, const float* k, const float* v, const float* out,
    const float* lse, const float* d_attn_out, float* d_q, float* d_k, float* d_v, int32_t seq_len,
    int32_t num_heads, int32_t head_dim, int32_t window_size, int32_t batch_size, int32_t n_persistent)
{
    int rc = sf_check("nlh_swa_backward_f32", seq_len, num_heads, head_dim, window_size, batch_size, n_persistent);
    if (rc != NLH_OK || batch_size == 0) return rc;
    if (!q || !k || !v || !out || !lse || !d_attn_out || !d_q || !d_k || !d_v) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_swa_backward_f32", "NULL pointer");
        return NLH_ERR_INVALID_ARG;
    }
    const long long rows = (long long)batch_size * num_heads * seq_len;
    const unsigned grid = (unsigned)((rows + SF_WARPS - 1) / SF_WARPS);
    const float scale = 1.0f / sqrtf((float)head_dim);
    const int w = window_size < seq_len ? window_size : seq_len;
    cudaStream_t st = current_stream();
    {
        const size_t smem = (size_t)SF_WARPS * (2 * head_dim + SF_MAX_KEYS) * sizeof(float);
        swa_f32_dq_kernel<<<grid, SF_WARPS * 32, smem, st>>>(q, k, v, out, lse, d_attn_out, d_q, seq_len,
            num_heads, head_dim, w, n_persistent, batch_size, scale);
        if (!check_launch("nlh_swa_backward_f32(dq)")) return NLH_ERR_CUDA;
    }
    {
        const size_t smem = (size_t)SF_WARPS * (2 * head_dim + 2 * SF_CHUNK) * sizeof(float);
        swa_f32_dkv_kernel<false><<<grid, SF_WARPS * 32, smem, st>>>(q, k, v, out, lse, d_attn_out, d_k, d_v,
            seq_len, num_heads, head_dim, w, n_persistent, batch_size, scale);
    }
    return check_launch("nlh_swa_backward_f32(dkv)") ? NLH_OK : NLH_ERR_CUDA;
}

}  // extern "C"
