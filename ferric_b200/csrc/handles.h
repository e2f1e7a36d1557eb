// The opaque handle types of the C ABI and small host helpers shared by the translation units
// that implement it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

struct ferric_cuda_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    uint64_t launches = 0;
    ferric::GemvTuning tune;
    cudaDeviceProp prop;
};

struct ferric_qmatrix {
    uint32_t ty = 0;
    int device = 0;
    ferric::DeviceWeights w;
    void* storage = nullptr;
    size_t storage_bytes = 0;
};

namespace ferric {

// Makes `dev` current for the scope of a call and restores the caller's device afterwards.
struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit DeviceGuard(int dev)
    {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard()
    {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// Grow the context's activation scratch (stream-ordered); defined in ffi.cu.
int32_t ensure_scratch(ferric_cuda_ctx* ctx, size_t bytes);

}  // namespace ferric
