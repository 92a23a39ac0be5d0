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
// Scratch is grow-only, per device and per SLOT. All launches use slot 0 unless the caller
// selects another one (nlh_set_workspace_slot): a caller that runs launches on several streams
// concurrently gives each stream its own slot so that they do not share scratch.
constexpr int WS_SLOTS = 8;
struct WsSlot {
    void* ptr;
    size_t bytes;
};
static int g_ws_slot = 0;
static WsSlot g_ws[MAX_DEVICES][WS_SLOTS] = {};

cudaStream_t current_stream() { return g_stream; }

// Library options (nlh_set_option); index = option id, all default to 1 (enabled).
constexpr int MAX_OPTIONS = 8;
static int g_options[MAX_OPTIONS] = {1, 1, 1, 1, 1, 1, 1, 1};
int option_value(int option) { return (option >= 0 && option < MAX_OPTIONS) ? g_options[option] : 0; }

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
    WsSlot* slot = &g_ws[dev][g_ws_slot];
    if (bytes <= slot->bytes && slot->ptr != nullptr) return slot->ptr;
    // cudaFree synchronises the device, so kernels still using the old block finish first.
    if (slot->ptr != nullptr) { cudaFree(slot->ptr); slot->ptr = nullptr; slot->bytes = 0; }
    size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
        record_status(NLH_ERR_WORKSPACE, "workspace cudaMalloc", cudaGetErrorString(e));
        return nullptr;
    }
    slot->ptr = p;
    slot->bytes = want;
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
    for (int i = 0; i < nlh::WS_SLOTS; i++) {
        nlh::WsSlot& s = nlh::g_ws[dev][i];
        if (s.ptr) cudaFree(s.ptr);
        s = nlh::WsSlot{};
    }
}
int64_t nlh_workspace_bytes(void)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= nlh::MAX_DEVICES) return -1;
    int64_t total = 0;
    for (int i = 0; i < nlh::WS_SLOTS; i++) total += (int64_t)nlh::g_ws[dev][i].bytes;
    return total;
}
int32_t nlh_set_workspace_slot(int32_t slot)
{
    if (slot < 0 || slot >= nlh::WS_SLOTS) return NLH_ERR_INVALID_ARG;
    nlh::g_ws_slot = slot;
    return NLH_OK;
}
int32_t nlh_set_option(int32_t option, int32_t value)
{
    if (option < 1 || option >= nlh::MAX_OPTIONS) return NLH_ERR_INVALID_ARG;
    nlh::g_options[option] = value ? 1 : 0;
    return NLH_OK;
}
int32_t nlh_abi_version(void) { return 1; }

// SimpleRng of the reference (core/src/tensor.rs:380-408), host side.
void nlh_simple_rng_fill(uint64_t* state, float scale, float* out_host, int64_t n)
{
    if (!state || !out_host || n <= 0) return;
    uint64_t s = *state == 0 ? 1 : *state;
    for (int64_t i = 0; i < n; i++) {
        s ^= s << 13;
        s ^= s >> 7;
        s ^= s << 17;
        const double u = (double)s / 18446744073709551615.0;
        out_host[i] = (2.0f * (float)u - 1.0f) * scale;
    }
    *state = s;
}

}  // extern "C"
