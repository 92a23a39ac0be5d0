// C-ABI form of the reference's opaque-VJP registry for the hot-path keys
// (core/src/tape.rs:98-145 OpaqueKey / OpaqueBackwardFn; adapters core/src/opaque_adapters.rs).
//
// The reference's Wengert tape holds HOST slices: an adapter receives the upstream gradients
// and the buffers saved by the forward and fills the input gradients. nlh_opaque_backward keeps
// that calling convention over plain pointers and runs the kernel-level adapters on the GPU:
//   DGD                 opaque_adapters.rs:1680-1725  saved [meta(seq,d[,clip]), k,v,q,alpha,theta,m_states]
//   SWA                 opaque_adapters.rs:952-997    saved [meta(seq,heads,head_dim,window), q,k,v,attn_weights]
//   Frozen{Delta,Titans,Hebbian} read
//                       opaque_adapters.rs:999-1069   saved [meta(seq,d), M]           d_q[t] = M^T d_y[t]
// The rule-level adapters (DeltaRule, TitansLMM, HebbianRule: projections, gates and the flat
// parameter vector inside one block) live in opaque_rules.cu; every key off the path returns
// NLH_ERR_UNSUPPORTED.
// Staging buffers are allocated and freed per call, like the reference's host-slice dispatch
// functions (core/src/dispatch.rs:330-1213).
#include <cuda_bf16.h>

#include "host_staging.cuh"
#include "../../include/nlh_ffi.h"

namespace nlh {

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = __float2bfloat16(src[i]);
}

// d_q[t, i] = sum_j M[j, i] * d_y[t, j]
__global__ void frozen_read_bwd_kernel(const float* __restrict__ m, const float* __restrict__ d_y,
                                       float* __restrict__ d_q, int seq, int d)
{
    const long long n = (long long)seq * d;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / d), i = (int)(idx - (long long)t * d);
        float s = 0.f;
        for (int j = 0; j < d; j++) s += m[(size_t)j * d + i] * d_y[(size_t)t * d + j];
        d_q[idx] = s;
    }
}

// opaque_rules.cu
int opaque_rule_backward(int rule, int n_out, const float* const* d_outputs, const int64_t* out_len,
                         int n_saved, const float* const* saved, const int64_t* saved_len, int n_in,
                         float* const* d_inputs, const int64_t* in_len);

static int fail(int code, const char* detail)
{
    record_status(code, "nlh_opaque_backward", detail);
    return code;
}

}  // namespace nlh

using namespace nlh;

extern "C" int32_t nlh_opaque_backward(int32_t key, int32_t n_out, const float* const* d_outputs,
    const int64_t* out_len, int32_t n_saved, const float* const* saved, const int64_t* saved_len,
    int32_t n_in, float* const* d_inputs, const int64_t* in_len)
{
    if (n_out < 1 || n_saved < 1 || n_in < 1 || !d_outputs || !out_len || !saved || !saved_len ||
        !d_inputs || !in_len || saved_len[0] < 2)
        return fail(NLH_ERR_INVALID_ARG, "need at least one output gradient, a meta buffer and one input gradient");
    cudaStream_t st = current_stream();
    const float* meta = saved[0];
    Staging sg;

    if (key == NLH_KEY_DELTA_RULE || key == NLH_KEY_TITANS_LMM || key == NLH_KEY_HEBBIAN_RULE) {
        const int rule = key == NLH_KEY_DELTA_RULE ? 0 : (key == NLH_KEY_TITANS_LMM ? 1 : 2);
        return opaque_rule_backward(rule, n_out, d_outputs, out_len, n_saved, saved, saved_len, n_in, d_inputs, in_len);
    }
    if (key == NLH_KEY_DGD) {
        const long long seq = (long long)meta[0], d = (long long)meta[1];
        const float clip = saved_len[0] > 2 ? meta[2] : 0.0f;
        if (n_saved < 7 || n_in < 6 || seq <= 0 || d <= 0 || out_len[0] != seq * d ||
            saved_len[1] != seq * d || saved_len[2] != seq * d || saved_len[3] != seq * d ||
            saved_len[4] != seq || saved_len[5] != seq || saved_len[6] != (seq + 1) * d * d ||
            in_len[0] != seq * d || in_len[1] != seq * d || in_len[2] != seq * d || in_len[3] != seq ||
            in_len[4] != seq || in_len[5] != d * d)
            return fail(NLH_ERR_INVALID_ARG, "DGD: buffer counts or lengths do not match meta (seq, d)");
        float* k = sg.upload(saved[1], seq * d, st);
        float* v = sg.upload(saved[2], seq * d, st);
        float* q = sg.upload(saved[3], seq * d, st);
        float* al = sg.upload(saved[4], seq, st);
        float* th = sg.upload(saved[5], seq, st);
        float* ms = sg.upload(saved[6], (seq + 1) * d * d, st);
        float* dy = sg.upload(d_outputs[0], seq * d, st);
        float* g[6];
        const long long glen[6] = {seq * d, seq * d, seq * d, seq, seq, d * d};
        for (int i = 0; i < 6; i++) g[i] = sg.zeros(glen[i], st);
        if (!sg.ok) return fail(NLH_ERR_CUDA, "DGD: device staging failed");
        nlh_clear_status();
        dgd_backward_f32_cuda(k, v, q, al, th, ms, dy, g[0], g[1], g[2], g[3], g[4], g[5], (int)seq, (int)d, clip);
        if (nlh_last_status() != NLH_OK) return nlh_last_status();
        for (int i = 0; i < 6; i++)
            if (!download(d_inputs[i], g[i], glen[i], st)) return fail(NLH_ERR_CUDA, "DGD: download failed");
    } else if (key == NLH_KEY_SWA) {
        if (saved_len[0] < 4) return fail(NLH_ERR_INVALID_ARG, "SWA: meta must hold seq, heads, head_dim, window");
        const long long seq = (long long)meta[0], nh = (long long)meta[1], hd = (long long)meta[2], w = (long long)meta[3];
        const long long n = seq * nh * hd;
        if (n_saved < 4 || n_in < 3 || seq <= 0 || nh <= 0 || hd <= 0 || w <= 0 || out_len[0] != n ||
            saved_len[1] != n || saved_len[2] != n || saved_len[3] != n || in_len[0] != n || in_len[1] != n || in_len[2] != n)
            return fail(NLH_ERR_INVALID_ARG, "SWA: buffer counts or lengths do not match meta");
        __nv_bfloat16* h16[3];
        for (int i = 0; i < 3; i++) {
            float* f = sg.upload(saved[1 + i], n, st);
            h16[i] = (__nv_bfloat16*)sg.alloc((size_t)n * sizeof(__nv_bfloat16));
            if (!sg.ok) return fail(NLH_ERR_CUDA, "SWA: device staging failed");
            f32_to_bf16_kernel<<<(unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096), 256, 0, st>>>(f, h16[i], n);
        }
        float* dout = sg.upload(d_outputs[0], n, st);
        float* g[3];
        for (int i = 0; i < 3; i++) g[i] = sg.zeros(n, st);
        if (!sg.ok || !check_launch("nlh_opaque_backward")) return fail(NLH_ERR_CUDA, "SWA: device staging failed");
        nlh_clear_status();
        swa_backward_f32_cuda((const uint16_t*)h16[0], (const uint16_t*)h16[1], (const uint16_t*)h16[2], nullptr,
                              dout, g[0], g[1], g[2], (int)seq, (int)nh, (int)hd, (int)w, 1, 0);
        if (nlh_last_status() != NLH_OK) return nlh_last_status();
        for (int i = 0; i < 3; i++)
            if (!download(d_inputs[i], g[i], n, st)) return fail(NLH_ERR_CUDA, "SWA: download failed");
    } else if (key == NLH_KEY_FROZEN_DELTA_RULE || key == NLH_KEY_FROZEN_TITANS_LMM || key == NLH_KEY_FROZEN_HEBBIAN_RULE) {
        const long long seq = (long long)meta[0], d = (long long)meta[1];
        if (saved_len[0] > 2 && meta[2] != 0.0f)
            return fail(NLH_ERR_UNSUPPORTED, "frozen read: only the identity feature map is on the path");
        if (saved_len[0] >= 7 && key == NLH_KEY_FROZEN_TITANS_LMM)   // extended meta = MLP memory tape
            return fail(NLH_ERR_UNSUPPORTED, "frozen read: MLP memory is not on the path");
        if (n_saved < 2 || seq <= 0 || d <= 0 || out_len[0] != seq * d || saved_len[1] != d * d || in_len[0] != seq * d)
            return fail(NLH_ERR_INVALID_ARG, "frozen read: buffer counts or lengths do not match meta (seq, d)");
        float* m = sg.upload(saved[1], d * d, st);
        float* dy = sg.upload(d_outputs[0], seq * d, st);
        float* dq = sg.zeros(seq * d, st);
        if (!sg.ok) return fail(NLH_ERR_CUDA, "frozen read: device staging failed");
        const long long n = seq * d;
        frozen_read_bwd_kernel<<<(unsigned)((n + 127) / 128 < 4096 ? (n + 127) / 128 : 4096), 128, 0, st>>>(m, dy, dq, (int)seq, (int)d);
        if (!check_launch("nlh_opaque_backward")) return NLH_ERR_CUDA;
        if (!download(d_inputs[0], dq, n, st)) return fail(NLH_ERR_CUDA, "frozen read: download failed");
    } else {
        return fail(NLH_ERR_UNSUPPORTED, "no GPU adapter for this key (it is off the path)");
    }
    if (cudaStreamSynchronize(st) != cudaSuccess) return fail(NLH_ERR_CUDA, "stream synchronisation failed");
    return NLH_OK;
}
