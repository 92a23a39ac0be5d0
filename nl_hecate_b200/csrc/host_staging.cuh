// Device staging of host slices for the host-pointer entries (one cudaMalloc per buffer, all
// released when the object dies — like the GpuBuf temporaries of core/src/dispatch.rs:1665-2090).
#pragma once

#include <vector>

#include "nlh_common.cuh"

namespace nlh {

struct Staging {
    std::vector<void*> bufs;
    bool ok = true;
    ~Staging() { for (void* p : bufs) cudaFree(p); }
    void* alloc(size_t bytes)
    {
        void* p = nullptr;
        if (bytes == 0) bytes = 4;
        if (cudaMalloc(&p, bytes) != cudaSuccess) { ok = false; return nullptr; }
        bufs.push_back(p);
        return p;
    }
    float* upload(const float* host, long long n, cudaStream_t st)
    {
        float* p = (float*)alloc((size_t)(n > 0 ? n : 1) * sizeof(float));
        if (p && n > 0 && cudaMemcpyAsync(p, host, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, st) != cudaSuccess) ok = false;
        return p;
    }
    float* zeros(long long n, cudaStream_t st)
    {
        float* p = (float*)alloc((size_t)(n > 0 ? n : 1) * sizeof(float));
        if (p && cudaMemsetAsync(p, 0, (size_t)(n > 0 ? n : 1) * sizeof(float), st) != cudaSuccess) ok = false;
        return p;
    }
    float* empty(long long n) { return (float*)alloc((size_t)(n > 0 ? n : 1) * sizeof(float)); }
};

inline bool download(float* host, const float* dev, long long n, cudaStream_t st)
{
    return n <= 0 || cudaMemcpyAsync(host, dev, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost, st) == cudaSuccess;
}

}  // namespace nlh
