// Titans LMM backward for callers that must not allocate device memory.
//
// Some hosts cannot let a library call cudaMalloc: they have handed the whole
// device to their own arena or buffer pool, so a stray allocation may fail or
// fragment it; or they sit in a latency-critical loop where the implicit
// device-wide synchronisation of cudaMalloc/cudaFree is not acceptable; or
// they run plug-ins under a policy that forbids allocation calls. The other
// backward entries of this library take their private scratch (the running
// d_M / d_S accumulators of the generic-d kernel) from a grow-only workspace
// that is cudaMalloc'ed on first use. This entry runs the same generic-d
// kernel with that scratch placed in a fixed array that is part of the
// library image instead, so it performs no allocation of any kind: no
// cudaMalloc, cudaFree, workspace growth or allocating library routine.
//
// Cost and limits:
//   * the array is NLH_NOALLOC_SCRATCH_BYTES (2 MiB) of device memory, held by
//     every GPU that loads the library until the process exits;
//   * batch_size * d * d must not exceed NLH_NOALLOC_MAX_STATE_FLOATS
//     (262144: e.g. 64 problems at d = 64, 16 at d = 128, one at d = 512);
//     larger requests are rejected with NLH_ERR_INVALID_ARG;
//   * all calls on a device share the one array. It keeps whatever the last
//     call left in it; the kernel re-initialises both accumulators (zero) at
//     its start, so calls issued one after another on one stream are
//     independent. Two calls that overlap on the GPU (different streams, or
//     different host threads with different streams) race on the array and
//     give wrong results: serialise them.
//   * s_states must be given: the M-only form of titans_backward_f32_cuda
//     (s_states == NULL) is not available here and is rejected on the host;
//   * the first call on each device looks up the device address of the array
//     (cudaGetSymbolAddress). Make that first call while the stream is not
//     being captured; later calls do no set-up work.
#include <mutex>

#include "memory_generic.cuh"
#include "../../include/nlh_ffi.h"

namespace {

constexpr size_t kMaxStateFloats = 262144;                 // per accumulator
constexpr int kMaxDevices = 64;

// d_M accumulators in [0, kMaxStateFloats), d_S accumulators behind them.
// In host code this name is only a handle for cudaGetSymbolAddress; it is never
// passed to a kernel directly.
static __device__ __align__(256) float g_noalloc_scratch[2 * kMaxStateFloats];

float* g_scratch_dev_ptr[kMaxDevices] = {nullptr};
std::mutex g_setup_mu;

// Device address of the array on the current device (looked up once per device).
int scratch_for_current_device(float** out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        nlh::record_status(NLH_ERR_CUDA, "nlh_titans_backward_noalloc", "cudaGetDevice failed");
        return NLH_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (g_scratch_dev_ptr[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            nlh::record_status(NLH_ERR_CUDA, "nlh_titans_backward_noalloc(cudaGetSymbolAddress)",
                               cudaGetErrorString(e));
            return NLH_ERR_CUDA;
        }
        g_scratch_dev_ptr[dev] = p;
    }
    *out = g_scratch_dev_ptr[dev];
    return NLH_OK;
}

}  // namespace

extern "C" int32_t nlh_titans_backward_noalloc(
    const float* k_mem, const float* v_mem, const float* q_mem, const float* alpha,
    const float* theta, const float* eta, const float* m_states, const float* s_states,
    const float* d_y, float* d_k_mem, float* d_v_mem, float* d_q_mem, float* d_alpha,
    float* d_theta, float* d_eta, float* d_m_initial, float* d_s_initial, int32_t seq_len,
    int32_t d, int32_t batch_size, float error_clip)
{
    using namespace nlh;
    if (d <= 0 || seq_len < 0 || batch_size < 0) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_titans_backward_noalloc",
                      "d must be > 0, seq_len and batch_size >= 0");
        return NLH_ERR_INVALID_ARG;
    }
    if (batch_size == 0) return NLH_OK;
    // Unlike titans_backward_f32_cuda this entry always reads the stored momentum trajectory:
    // the kernel behind it has no M-only mode, so s_states must not be NULL. Every other pointer
    // is dereferenced on the device as well; reject NULL here instead of faulting there.
    if (!k_mem || !v_mem || !q_mem || !alpha || !theta || !eta || !m_states || !s_states || !d_y ||
        !d_k_mem || !d_v_mem || !d_q_mem || !d_alpha || !d_theta || !d_eta || !d_m_initial ||
        !d_s_initial) {
        record_status(NLH_ERR_INVALID_ARG, "nlh_titans_backward_noalloc",
                      "NULL pointer argument (this entry needs every buffer, including the stored "
                      "s_states trajectory)");
        return NLH_ERR_INVALID_ARG;
    }
    const size_t need = (size_t)batch_size * (size_t)d * (size_t)d;
    if (need > kMaxStateFloats) {
        char msg[160];
        snprintf(msg, sizeof(msg),
                 "batch_size*d*d = %zu exceeds the built-in scratch of %zu floats per accumulator; "
                 "use titans_backward_f32_cuda (allocating) for this size", need, kMaxStateFloats);
        record_status(NLH_ERR_INVALID_ARG, "nlh_titans_backward_noalloc", msg);
        return NLH_ERR_INVALID_ARG;
    }
    float* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != NLH_OK) return rc;

    BwdArgs a;
    a.k = k_mem; a.v = v_mem; a.q = q_mem; a.alpha = alpha; a.theta = theta; a.eta = eta;
    a.m_traj = m_states; a.s_traj = s_states; a.d_y = d_y;
    a.d_m_seed = nullptr; a.d_s_seed = nullptr;
    a.d_k = d_k_mem; a.d_v = d_v_mem; a.d_q = d_q_mem;
    a.d_alpha = d_alpha; a.d_theta = d_theta; a.d_eta = d_eta;
    a.d_m_out = d_m_initial; a.d_s_out = d_s_initial;
    a.dM = scratch;                       // zeroed by the kernel before use
    a.dS = scratch + kMaxStateFloats;     // zeroed by the kernel before use
    a.dM0 = nullptr; a.m_rec = nullptr; a.s_rec = nullptr;
    a.seq_len = seq_len; a.d = d; a.batch = batch_size;
    a.t_start = 0; a.t_end = seq_len;
    a.traj_stride = (long long)(seq_len + 1) * d * d;
    a.frozen = 0; a.chunk = 0;
    a.atomic_out = 1;                     // summed over the batch, like titans_backward_f32_cuda
    a.error_clip = error_clip; a.m_norm_max = 0.0f;

    // d*d <= 262144 bounds d at 512, so the dynamic shared memory stays far below the
    // 48 KiB default and no function attribute has to be raised.
    const size_t smem = gen_bwd_smem(d);
    gen_bwd_kernel<RULE_TITANS><<<batch_size, GEN_THREADS, smem, current_stream()>>>(a);
    return check_launch("nlh_titans_backward_noalloc") ? NLH_OK : NLH_ERR_CUDA;
}
