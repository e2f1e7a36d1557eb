// The opaque handle types of the C ABI and small host helpers shared by the translation units
// that implement it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>

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
    // chained products (ferric_cuda_chain_*): the scratch holds two prepared-activation slots, slot 1 at this offset
    // (0 until ferric_cuda_chain_reserve); sums of squares, block tickets and the job counter live beside the split workspace
    size_t chain_slot_bytes = 0;
    // profiling buckets (ferric_cuda_prof / _prof_report): label -> milliseconds, and the previous mark
    bool prof_on = false, prof_marked = false;
    double prof_prev_ms = 0.0;
    std::map<std::string, double> prof;
    float* chain_ssq = nullptr;
    unsigned* chain_tickets = nullptr;
    unsigned* chain_done = nullptr;
};

struct ferric_qmatrix {
    uint32_t ty = 0;
    int device = 0;
    ferric::DeviceWeights w;
    void* storage = nullptr;
    size_t storage_bytes = 0;
};

// Proj (crates/ferric-llama/src/qwen3.rs:192-228): one logical projection whose stacked outputs live in one matrix
// (Fused: a single part) or, when the parts' quant formats differ, in one matrix per part (Split).
struct ferric_proj {
    ferric_qmatrix* parts[8] = {};
    size_t n_parts = 0, rows = 0, cols = 0;
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

struct ferric_chain_link;

namespace ferric {

// Argument checks of a chain link and the Chain record for its launch (the exchange parts are the caller's); defined
// in ffi.cu.
int32_t chain_setup(ferric_cuda_ctx* ctx, const ferric_chain_link* link, size_t m, bool pushed, Chain* chain,
                    const void** frag_in, Epilogue* epi, size_t* ldy);

}  // namespace ferric
