// Shared device helpers: error plumbing, f16 bit tricks, the m16n8k16 tensor-core wrapper.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "layout.h"

namespace ferric {

// Status codes of the C ABI (mirrored in include/ferric_cuda.h).
enum : int32_t {
    kOk = 0,
    kErrInvalidArg = 1,
    kErrUnsupportedType = 2,
    kErrShape = 3,
    kErrCuda = 4,
    kErrOom = 5,
    kUnsupported = 6,
    kErrTimeout = 7,
};

void set_last_error(const char* fmt, ...);
int32_t cuda_fail(cudaError_t e, const char* what);

#define FERRIC_CUDA_TRY(expr)                                        \
    do {                                                             \
        cudaError_t _e = (expr);                                     \
        if (_e != cudaSuccess) return ::ferric::cuda_fail(_e, #expr); \
    } while (0)

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Multiply two packed f16 pairs given as raw bits.  Subnormal operands and results are kept (no
// flush to zero): the GEMV kernels carry small integers as q * 2^-24 and rely on exact products.
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col).
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 128-bit streaming load of weight bytes: read-only path, evict-first in L1 so the one-pass weight
// stream does not push the (re-used) activation fragments out.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const void* p)
{
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Two unsigned bytes of `w` (selected by a PRMT byte selector with zero fill) as a packed pair of
// f16 integers: byte -> (0x6400 | byte) = 1024 + byte, then minus 1024.
__device__ __forceinline__ uint32_t bytes_to_h2(uint32_t w, uint32_t sel)
{
    uint32_t biased = __byte_perm(w, 0x64646464u, sel);
    return h2_as_u32(__hsub2(u32_as_h2(biased), u32_as_h2(0x64006400u)));
}

// Programmatic dependent launch.  Every hot-path kernel lets its successor in the stream start
// launching at once (launch_dependents) and blocks (wait) before it touches anything an earlier
// kernel produces or still reads.  A successor therefore overlaps its launch latency and its
// weight prefetch -- weights are immutable -- with the tail of its predecessor.  Every kernel
// executes the wait, so completion order stays transitive along the stream.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Loads of activations and activation fragments: data another kernel wrote, possibly while this
// kernel was already resident (it only *used* them after pdl_wait).  They must take the coherent
// path -- never ld.global.nc, whose lines may predate the producer's writes.
__device__ __forceinline__ uint2 ld_act(const uint2* p)
{
    uint2 v;
    asm volatile("ld.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_act(const float4* p)
{
    float4 v;
    asm volatile("ld.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                                 Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same launch with the grid cut into thread-block clusters of `cluster_x` CTAs along x.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                                         unsigned cluster_x, Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

}  // namespace ferric
