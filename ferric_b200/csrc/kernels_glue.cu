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

// The same with 16-byte accesses (d a multiple of 4, buffers 16-byte aligned): a row of up to 4 * KEEP * 512 floats stays
// in registers between the two passes, so a many-row batch reads its inputs once.
template <int KEEP>
__global__ void __launch_bounds__(512) add_rmsnorm_vec_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                              const float* __restrict__ w, float eps, size_t d4,
                                                              float* __restrict__ sum, float* __restrict__ norm)
{
    __shared__ float part[16];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = blockIdx.x * d4;
    const float4* a4 = reinterpret_cast<const float4*>(a) + base;
    const float4* b4 = b ? reinterpret_cast<const float4*>(b) + base : nullptr;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    float4* s4 = sum ? reinterpret_cast<float4*>(sum) + base : nullptr;
    float4* n4 = reinterpret_cast<float4*>(norm) + base;
    auto form = [&](size_t j) {
        float4 s = a4[j];
        if (b4) {
            const float4 t = b4[j];
            s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
        }
        return s;
    };
    auto scaled = [&](const float4& s, float inv, size_t j) {
        float4 o = make_float4(s.x * inv, s.y * inv, s.z * inv, s.w * inv);
        if (w4) {
            const float4 g = __ldg(w4 + j);
            o.x *= g.x; o.y *= g.y; o.z *= g.z; o.w *= g.w;
        }
        return o;
    };
    float4 keep[KEEP];
    float ms = 0.0f;
#pragma unroll
    for (int k = 0; k < KEEP; k++) {
        const size_t j = threadIdx.x + (size_t)k * blockDim.x;
        keep[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < d4) {
            keep[k] = form(j);
            if (s4) s4[j] = keep[k];
            ms = fmaf(keep[k].x, keep[k].x, fmaf(keep[k].y, keep[k].y, fmaf(keep[k].z, keep[k].z, fmaf(keep[k].w, keep[k].w, ms))));
        }
    }
    for (size_t j = threadIdx.x + (size_t)KEEP * blockDim.x; j < d4; j += blockDim.x) {
        const float4 s = form(j);
        if (s4) s4[j] = s;
        ms = fmaf(s.x, s.x, fmaf(s.y, s.y, fmaf(s.z, s.z, fmaf(s.w, s.w, ms))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ms += __shfl_xor_sync(0xffffffffu, ms, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ms;
    __syncthreads();
    float tot = 0.0f;
    for (int i = 0; i < (int)(blockDim.x >> 5); i++) tot += part[i];
    const float inv = 1.0f / sqrtf(tot / (float)(4 * d4) + eps);
#pragma unroll
    for (int k = 0; k < KEEP; k++) {
        const size_t j = threadIdx.x + (size_t)k * blockDim.x;
        if (j < d4) n4[j] = scaled(keep[k], inv, j);
    }
    for (size_t j = threadIdx.x + (size_t)KEEP * blockDim.x; j < d4; j += blockDim.x)
        n4[j] = scaled(s4 ? s4[j] : form(j), inv, j);   // (the sum may alias `a`: re-form it as the first pass did)
}

int32_t launch_add_rmsnorm(cudaStream_t st, const float* a, const float* b, const float* weight, float eps,
                           size_t rows, size_t d, float* sum, float* norm, const GemvTuning& tune)
{
    if (rows == 0 || d == 0) return kOk;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(weight) |
                           reinterpret_cast<uintptr_t>(sum) | reinterpret_cast<uintptr_t>(norm);
    if (d % 4 == 0 && (bits & 15) == 0) {
        const size_t d4 = d / 4;
        unsigned threads = (unsigned)((d4 + 3) / 4 + 31) / 32 * 32;   // the row in four register slots per thread where it fits
        if (threads < 64) threads = 64;
        if (threads > 512) threads = 512;
        FERRIC_CUDA_TRY(launch_kernel(add_rmsnorm_vec_kernel<4>, dim3((unsigned)rows), dim3(threads), 0, st, tune.pdl, a, b, weight, eps,
                                      d4, sum, norm));
        return kOk;
    }
    FERRIC_CUDA_TRY(launch_kernel(add_rmsnorm_kernel, dim3((unsigned)rows), dim3(256), 0, st, tune.pdl, a, b, weight, eps, d,
                                  sum, norm));
    return kOk;
}

}  // namespace ferric
