// The step either side of the matmuls in a decoder layer: fused residual add + RMSNorm
// (crates/ferric-tensor/src/lib.rs:372-384 and kernels :2018-2032, :2057-2075).  One CTA per row.
#include "common.cuh"
#include "kernels.h"

namespace ferric {

__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                          const float* __restrict__ w, float eps, size_t d,
                                                          float* __restrict__ sum, float* __restrict__ norm)
{
    __shared__ float part[8];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = blockIdx.x * d;
    float ms = 0.0f;
    for (size_t j = threadIdx.x; j < d; j += blockDim.x) {
        float s = a[base + j] + (b ? b[base + j] : 0.0f);
        if (sum) sum[base + j] = s;
        ms = fmaf(s, s, ms);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ms += __shfl_xor_sync(0xffffffffu, ms, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ms;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += part[i];
    const float inv = 1.0f / sqrtf(tot / (float)d + eps);
    for (size_t j = threadIdx.x; j < d; j += blockDim.x) {
        // re-form the sum exactly as the first pass did (it may alias `a` through `sum`)
        float s = sum ? sum[base + j] : a[base + j] + (b ? b[base + j] : 0.0f);
        norm[base + j] = s * inv * (w ? w[j] : 1.0f);
    }
}

int32_t launch_add_rmsnorm(cudaStream_t st, const float* a, const float* b, const float* weight, float eps,
                           size_t rows, size_t d, float* sum, float* norm, const GemvTuning& tune)
{
    if (rows == 0 || d == 0) return kOk;
    FERRIC_CUDA_TRY(launch_kernel(add_rmsnorm_kernel, dim3((unsigned)rows), dim3(256), 0, st, tune.pdl, a, b, weight, eps, d,
                                  sum, norm));
    return kOk;
}

}  // namespace ferric
