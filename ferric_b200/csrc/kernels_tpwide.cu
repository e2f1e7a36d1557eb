// All-reduce of a whole activation matrix (many rows: the batched decode path) by this library's own kernels over
// peer-mapped memory, in two pushed steps, fused at its end into the residual add + RMSNorm the layer runs next.
//
//   scatter:  every rank cuts its f32 partial [n] into `world` slices and stores slice s, as (value, exchange
//             number) pairs, into rank s's stage-1 region for this source rank;
//   reduce:   rank s polls the `world` copies of its slice in its own memory, adds them in rank order and stores the
//             sums, again as pairs, into the stage-2 region of every rank at the slice's place;
//   consume:  add + RMSNorm reads `b` from the stage-2 pairs in its own memory, polling each.
//
// Each element crosses NVLink twice (once per step) instead of `world - 1` times, every wait is a bounded poll on local
// memory for data that an earlier kernel of some rank stores, and an 8-byte store arrives whole, so a pair whose
// number matches carries its value.  No multicast, no multimem: plain stores to peer addresses.
#include "common.cuh"
#include "kernels.h"
#include "tpwide.cuh"

namespace ferric {

namespace {


// x[n] -> slice s of every four-float group goes to rank s (slices of `slice` floats, a multiple of 4).
__global__ void __launch_bounds__(256) wide_scatter_kernel(const float* __restrict__ x, size_t n, WideDst dst)
{
    pdl_launch_dependents();
    pdl_wait();
    const unsigned stamp = wide_stamp(dst.epoch);
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    const size_t owner = i / dst.slice, off = i - owner * dst.slice;
    uint2* base = nullptr;
#pragma unroll
    for (int r = 0; r < kMaxRanks; r++)
        if ((size_t)r == owner) base = dst.stage1[r];   // static indices keep the table in the parameter space
    store_pairs4(base + (size_t)(stamp & 1) * dst.parity_stride1 + off, v, stamp);
}

// This rank's slice: poll every source's copy, add in rank order, store the sums to every rank.
__global__ void __launch_bounds__(256) wide_reduce_kernel(size_t n, WideDst dst)
{
    pdl_launch_dependents();
    pdl_wait();
    const unsigned stamp = wide_stamp(dst.epoch);
    const size_t first = (size_t)dst.rank * dst.slice;
    const size_t len = first >= n ? 0 : (n - first < dst.slice ? n - first : dst.slice);
    const size_t off = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (off >= len) return;
    const uint2* mine = dst.recv1 + (size_t)(stamp & 1) * dst.parity_stride1 + off;   // [source rank][slice]
    const int limit = *reinterpret_cast<volatile int*>(dst.status) ? 0 : dst.wait_spins;
    uint4 a[kMaxRanks], b[kMaxRanks];
    int spins = 0;
    for (;;) {
#pragma unroll
        for (int r = 0; r < kMaxRanks; r++)
            if (r < dst.world) load_pairs4(mine + (size_t)r * dst.slice, a[r], b[r]);
        bool ok = true;
#pragma unroll
        for (int r = 0; r < kMaxRanks; r++)
            if (r < dst.world) ok = ok && a[r].y == stamp && a[r].w == stamp && b[r].y == stamp && b[r].w == stamp;
        if (ok) break;
        if (++spins > limit) {
            *dst.status = 1;
            break;
        }
    }
    float4 s = make_float4(__uint_as_float(a[0].x), __uint_as_float(a[0].z), __uint_as_float(b[0].x), __uint_as_float(b[0].z));
#pragma unroll
    for (int r = 1; r < kMaxRanks; r++) {
        if (r < dst.world) {
            s.x += __uint_as_float(a[r].x); s.y += __uint_as_float(a[r].z);
            s.z += __uint_as_float(b[r].x); s.w += __uint_as_float(b[r].z);
        }
    }
    const size_t at = (size_t)(stamp & 1) * dst.parity_stride2 + first + off;
#pragma unroll
    for (int r = 0; r < kMaxRanks; r++)
        if (r < dst.world) store_pairs4(dst.stage2[r] + at, s, stamp);
}

// (sum, norm) = add_rmsnorm(a, b) with b polled from this rank's stage-2 pairs; one CTA per row.  The last CTA to
// finish closes the exchange.
__global__ void __launch_bounds__(256) wide_add_rmsnorm_kernel(const float* __restrict__ a, const float* __restrict__ w, float eps,
                                                               size_t d, float* __restrict__ sum, float* __restrict__ norm,
                                                               WideDst dst)
{
    __shared__ float part[8];
    pdl_launch_dependents();
    pdl_wait();
    const unsigned stamp = wide_stamp(dst.epoch);
    const int limit = *reinterpret_cast<volatile int*>(dst.status) ? 0 : dst.wait_spins;
    const size_t base = blockIdx.x * d;
    const uint2* pairs = dst.recv2 + (size_t)(stamp & 1) * dst.parity_stride2 + base;
    float ms = 0.0f;
    // the row's sums stay in registers between the two passes where they fit (kKeep quads per thread: d <= 8192 at 256 threads)
    constexpr int kKeep = 8;
    float4 keep[kKeep];
    auto consume = [&](size_t j) {
        uint4 pa, pb;
        int spins = 0;
        for (;;) {
            load_pairs4(pairs + j, pa, pb);
            if (pa.y == stamp && pa.w == stamp && pb.y == stamp && pb.w == stamp) break;
            if (++spins > limit) {
                *dst.status = 1;
                break;
            }
        }
        const float4 av = *reinterpret_cast<const float4*>(a + base + j);
        const float4 s = make_float4(av.x + __uint_as_float(pa.x), av.y + __uint_as_float(pa.z), av.z + __uint_as_float(pb.x),
                                     av.w + __uint_as_float(pb.z));
        *reinterpret_cast<float4*>(sum + base + j) = s;
        ms = fmaf(s.x, s.x, ms); ms = fmaf(s.y, s.y, ms); ms = fmaf(s.z, s.z, ms); ms = fmaf(s.w, s.w, ms);
        return s;
    };
#pragma unroll
    for (int k = 0; k < kKeep; k++) {
        const size_t j = ((size_t)k * blockDim.x + threadIdx.x) * 4;
        keep[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < d) keep[k] = consume(j);
    }
    for (size_t j = ((size_t)kKeep * blockDim.x + threadIdx.x) * 4; j < d; j += (size_t)blockDim.x * 4) (void)consume(j);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ms += __shfl_xor_sync(0xffffffffu, ms, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ms;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += part[i];
    const float inv = 1.0f / sqrtf(tot / (float)d + eps);
    if (norm) {
        auto emit = [&](size_t j, const float4& s) {
            float4 wv = make_float4(1.f, 1.f, 1.f, 1.f);
            if (w) wv = *reinterpret_cast<const float4*>(w + j);
            *reinterpret_cast<float4*>(norm + base + j) = make_float4(s.x * inv * wv.x, s.y * inv * wv.y, s.z * inv * wv.z, s.w * inv * wv.w);
        };
#pragma unroll
        for (int k = 0; k < kKeep; k++) {
            const size_t j = ((size_t)k * blockDim.x + threadIdx.x) * 4;
            if (j < d) emit(j, keep[k]);
        }
        for (size_t j = ((size_t)kKeep * blockDim.x + threadIdx.x) * 4; j < d; j += (size_t)blockDim.x * 4)
            emit(j, *reinterpret_cast<const float4*>(sum + base + j));   // this thread's own stores
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(dst.ticket, 1u) == gridDim.x - 1) {
            *dst.ticket = 0;
            asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(dst.epoch), "r"(stamp) : "memory");
        }
    }
}

}  // namespace

int32_t launch_wide_allreduce_add_rmsnorm(cudaStream_t st, const float* partial, const float* a, const float* weight, float eps,
                                          size_t rows, size_t d, float* sum, float* norm, const WideDst& dst,
                                          const GemvTuning& tune, int steps)
{
    const size_t n = rows * d;
    if (n == 0) return kOk;
    const unsigned quads = (unsigned)((n + 3) / 4), slice_quads = (unsigned)(dst.slice / 4);
    if (steps & 1)
        FERRIC_CUDA_TRY(launch_kernel(wide_scatter_kernel, dim3((quads + 255) / 256), dim3(256), 0, st, tune.pdl, partial, n, dst));
    if (steps & 2)
        FERRIC_CUDA_TRY(launch_kernel(wide_reduce_kernel, dim3((slice_quads + 255) / 256), dim3(256), 0, st, tune.pdl, n, dst));
    if (steps & 4)
        FERRIC_CUDA_TRY(launch_kernel(wide_add_rmsnorm_kernel, dim3((unsigned)rows), dim3(256), 0, st, tune.pdl, a, weight, eps, d, sum,
                                      norm, dst));
    return kOk;
}

}  // namespace ferric
