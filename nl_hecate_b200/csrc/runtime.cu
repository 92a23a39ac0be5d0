// Library runtime: launch stream, recorded status, grow-only scratch.
#include "nlh_common.cuh"
#include "../../include/nlh_ffi.h"

#include <mutex>
#include <string>
#include <string.h>

namespace nlh {

static cudaStream_t g_stream = 0;
static int g_status = NLH_OK;
static char g_error[512] = "";
static std::mutex g_mu;

constexpr int MAX_DEVICES = 64;
static void* g_ws[MAX_DEVICES] = {nullptr};
static size_t g_ws_bytes[MAX_DEVICES] = {0};

cudaStream_t current_stream() { return g_stream; }

void record_status(int status, const char* where, const char* detail)
{
    std::lock_guard<std::mutex> lk(g_mu);
    g_status = status;
    snprintf(g_error, sizeof(g_error), "%s: %s", where ? where : "?", detail ? detail : "");
    fprintf(stderr, "[nlh_b200] error %d in %s\n", status, g_error);
}

void* workspace(size_t bytes)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        record_status(NLH_ERR_WORKSPACE, "workspace", "cudaGetDevice failed");
        return nullptr;
    }
    if (bytes <= g_ws_bytes[dev] && g_ws[dev] != nullptr) return g_ws[dev];
    // cudaFree synchronises the device, so kernels still using the old block finish first.
    if (g_ws[dev] != nullptr) { cudaFree(g_ws[dev]); g_ws[dev] = nullptr; g_ws_bytes[dev] = 0; }
    size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
        record_status(NLH_ERR_WORKSPACE, "workspace cudaMalloc", cudaGetErrorString(e));
        return nullptr;
    }
    g_ws[dev] = p;
    g_ws_bytes[dev] = want;
    return p;
}

}  // namespace nlh

extern "C" {

void nlh_set_stream(void* s) { nlh::g_stream = (cudaStream_t)s; }
void* nlh_get_stream(void) { return (void*)nlh::g_stream; }
int32_t nlh_last_status(void) { return nlh::g_status; }
const char* nlh_last_error(void) { return nlh::g_error; }
void nlh_clear_status(void) { nlh::g_status = NLH_OK; nlh::g_error[0] = 0; }
int32_t nlh_workspace_reserve(int64_t bytes)
{
    if (bytes < 0) return NLH_ERR_INVALID_ARG;
    return nlh::workspace((size_t)bytes) != nullptr ? NLH_OK : NLH_ERR_WORKSPACE;
}
void nlh_workspace_release(void)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= nlh::MAX_DEVICES) return;
    if (nlh::g_ws[dev]) { cudaFree(nlh::g_ws[dev]); nlh::g_ws[dev] = nullptr; nlh::g_ws_bytes[dev] = 0; }
}
int32_t nlh_abi_version(void) { return 1; }

}  // extern "C"
