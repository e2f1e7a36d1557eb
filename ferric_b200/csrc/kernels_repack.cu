// Load-time layout transform (raw GGUF block bytes -> device layout) and the bit-exact dequantisers.
//
// Repack replaces Q4_KWeights / Q6_KWeights / Q8_0Weights::from_bytes of the reference
// (crates/ferric-tensor/src/dtype.rs:1388-1420, :1147-1166, :1270-1286).  The dequantisers are
// the device twins of deq_q4_k / deq_q6_k / deq_q8_0 (crates/ferric-gguf/src/lib.rs:793-825,
// :721-746, :608-615): same operation order, every multiply and subtract rounded separately, so
// the f32 result is bit-identical to the reference's CPU decoders.
#include "common.cuh"
#include "kernels.h"

namespace ferric {

// ------------------------------------------------------------------------------- repack
// `src` addresses block (row0 + r, blk0 + b) of a raw matrix with src_nblk blocks per row, so a
// tensor-parallel shard (a row range or a K range) is re-packed straight out of the full tensor.

__global__ void repack_q4k_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, size_t nrows,
                                  size_t nblk, size_t src_nblk, size_t row0, size_t blk0, bool aligned)
{
    // 18 pieces of 8 bytes per block: the layout keeps every aligned 8-byte run contiguous
    size_t total = nrows * nblk * 18;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t c = i % 18, rb = i / 18, b = rb % nblk, r = rb / nblk;
        const uint8_t* s = src + ((row0 + r) * src_nblk + blk0 + b) * kQ4KBlock + 8 * c;
        uint8_t* d = dst + ((r >> 4) * nblk + b) * kQ4KUnit + q4k_unit_offset((int)(r & 15), (int)(8 * c));
        if (aligned) {
            *reinterpret_cast<uint2*>(d) = *reinterpret_cast<const uint2*>(s);
        } else {
            for (int j = 0; j < 8; j++) d[j] = s[j];
        }
    }
}

__global__ void repack_q5k_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, size_t nrows,
                                  size_t nblk, size_t src_nblk, size_t row0, size_t blk0)
{
    // 22 pieces of 8 bytes per block (header 2, fifth bits 4, nibbles 16); every aligned 8-byte run stays contiguous
    size_t total = nrows * nblk * 22;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t c = i % 22, rb = i / 22, b = rb % nblk, r = rb / nblk;
        const uint8_t* s = src + ((row0 + r) * src_nblk + blk0 + b) * kQ5KBlock + 8 * c;
        uint8_t* d = dst + ((r >> 4) * nblk + b) * kQ5KUnit + q5k_unit_offset((int)(r & 15), (int)(8 * c));
        for (int j = 0; j < 8; j++) d[j] = s[j];
    }
}

__global__ void repack_q6k_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, size_t nrows,
                                  size_t nblk, size_t src_nblk, size_t row0, size_t blk0)
{
    // 48 four-byte pieces of ql / qh (contiguous in both layouts) + one piece for scales and d
    size_t total = nrows * nblk * 49;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t p = i % 49, rb = i / 49, b = rb % nblk, r = rb / nblk;
        const uint8_t* s = src + ((row0 + r) * src_nblk + blk0 + b) * kQ6KBlock;
        uint8_t* u = dst + ((r >> 4) * nblk + b) * kQ6KUnit;
        int rr = (int)(r & 15);
        if (p < 48) {
            int byte0 = (int)(4 * p);
            uint32_t w = (uint32_t)s[byte0] | ((uint32_t)s[byte0 + 1] << 8) | ((uint32_t)s[byte0 + 2] << 16) |
                         ((uint32_t)s[byte0 + 3] << 24);
            *reinterpret_cast<uint32_t*>(u + q6k_unit_offset(rr, byte0)) = w;
        } else {
            for (int byte = 192; byte < 210; byte++) u[q6k_unit_offset(rr, byte)] = s[byte];
        }
    }
}

__global__ void repack_q8_0_kernel(const uint8_t* __restrict__ src, int8_t* __restrict__ qs,
                                   uint16_t* __restrict__ dplane, size_t nrows, size_t nb, size_t src_nb,
                                   size_t row0, size_t blk0)
{
    size_t total = nrows * nb;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t b = i % nb, r = i / nb;
        const uint8_t* s = src + ((row0 + r) * src_nb + blk0 + b) * kQ8Block;
        dplane[r * nb + b] = (uint16_t)(s[0] | (s[1] << 8));
        uint32_t w[8];
        for (int k = 0; k < 8; k++)
            w[k] = (uint32_t)s[2 + 4 * k] | ((uint32_t)s[3 + 4 * k] << 8) | ((uint32_t)s[4 + 4 * k] << 16) |
                   ((uint32_t)s[5 + 4 * k] << 24);
        uint4* d = reinterpret_cast<uint4*>(qs + (r * nb + b) * 32);
        d[0] = make_uint4(w[0], w[1], w[2], w[3]);
        d[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
}

static int grid_for(size_t total, int block)
{
    size_t g = (total + block - 1) / block;
    if (g > 148 * 64) g = 148 * 64;
    if (g < 1) g = 1;
    return (int)g;
}

int32_t launch_repack(cudaStream_t st, uint32_t ty, const uint8_t* src, DeviceWeights& w, size_t src_nblk,
                      size_t row0, size_t blk0)
{
    size_t nrows = w.rows, nblk = w.nblk;
    if (nrows == 0 || nblk == 0) return kOk;
    if (ty == kGgmlQ4K) {
        bool aligned = (reinterpret_cast<uintptr_t>(src) & 7) == 0;
        repack_q4k_kernel<<<grid_for(nrows * nblk * 18, 256), 256, 0, st>>>(src, w.units, nrows, nblk, src_nblk,
                                                                            row0, blk0, aligned);
    } else if (ty == kGgmlQ5K) {
        repack_q5k_kernel<<<grid_for(nrows * nblk * 22, 256), 256, 0, st>>>(src, w.units, nrows, nblk, src_nblk, row0, blk0);
    } else if (ty == kGgmlQ6K) {
        repack_q6k_kernel<<<grid_for(nrows * nblk * 49, 256), 256, 0, st>>>(src, w.units, nrows, nblk, src_nblk,
                                                                             row0, blk0);
    } else {
        repack_q8_0_kernel<<<grid_for(nrows * nblk, 256), 256, 0, st>>>(src, w.q8_qs, w.q8_d, nrows, nblk,
                                                                         src_nblk, row0, blk0);
    }
    FERRIC_CUDA_TRY(cudaGetLastError());
    return kOk;
}

// ------------------------------------------------------------------------------- dequant
// Byte accessors: the same decoder body runs on raw GGUF bytes (deq_raw) and on the device
// layout of a loaded matrix.

struct RawBytes {
    const uint8_t* p;
    size_t nblk, block;
    __device__ uint8_t at(size_t row, size_t blk, int byte) const { return p[(row * nblk + blk) * block + byte]; }
};
struct UnitQ4K {
    const uint8_t* p;
    size_t nblk, block;
    __device__ uint8_t at(size_t row, size_t blk, int byte) const
    {
        return p[((row >> 4) * nblk + blk) * kQ4KUnit + q4k_unit_offset((int)(row & 15), byte)];
    }
};
struct UnitQ5K {
    const uint8_t* p;
    size_t nblk, block;
    __device__ uint8_t at(size_t row, size_t blk, int byte) const
    {
        return p[((row >> 4) * nblk + blk) * kQ5KUnit + q5k_unit_offset((int)(row & 15), byte)];
    }
};
struct UnitQ6K {
    const uint8_t* p;
    size_t nblk, block;
    __device__ uint8_t at(size_t row, size_t blk, int byte) const
    {
        return p[((row >> 4) * nblk + blk) * kQ6KUnit + q6k_unit_offset((int)(row & 15), byte)];
    }
};
struct PlanesQ8 {
    const int8_t* qs;
    const uint16_t* d;
    size_t nblk, block;
    __device__ uint8_t at(size_t row, size_t blk, int byte) const
    {
        if (byte < 2) return (uint8_t)(d[row * nblk + blk] >> (8 * byte));
        return (uint8_t)qs[(row * nblk + blk) * 32 + (byte - 2)];
    }
};

__device__ __forceinline__ float f16_bits_to_f32(uint32_t lo, uint32_t hi)
{
    return __half2float(__ushort_as_half((unsigned short)(lo | (hi << 8))));
}

// crates/ferric-tensor/src/dtype.rs:4159-4163
__device__ __forceinline__ uint16_t bf16_rne_bits(float x)
{
    uint32_t b = __float_as_uint(x);
    uint32_t r = b + 0x7fffu + ((b >> 16) & 1u);
    return (uint16_t)(r >> 16);
}

template <class Acc>
__device__ float deq_elem_q4k(const Acc& a, size_t row, size_t col)
{
    size_t blk = col >> 8;
    int w = (int)(col & 255), grp = w >> 6, n = (w >> 5) & 1, l = w & 31;
    float d = f16_bits_to_f32(a.at(row, blk, 0), a.at(row, blk, 1));
    float dmin = f16_bits_to_f32(a.at(row, blk, 2), a.at(row, blk, 3));
    int j = 2 * grp + n;
    uint32_t sc, mn;
    if (j < 4) {
        sc = a.at(row, blk, 4 + j) & 63;
        mn = a.at(row, blk, 4 + j + 4) & 63;
    } else {
        uint32_t hi4 = a.at(row, blk, 4 + j + 4);
        sc = (hi4 & 0x0F) | ((a.at(row, blk, 4 + j - 4) >> 6) << 4);
        mn = (hi4 >> 4) | ((a.at(row, blk, 4 + j) >> 6) << 4);
    }
    uint32_t qb = a.at(row, blk, 16 + 32 * grp + l);
    uint32_t q = n ? (qb >> 4) : (qb & 0x0F);
    float d1 = __fmul_rn(d, (float)sc), mm = __fmul_rn(dmin, (float)mn);
    return __fsub_rn(__fmul_rn(d1, (float)q), mm);
}

// crates/ferric-gguf/src/lib.rs:690-716
template <class Acc>
__device__ float deq_elem_q5k(const Acc& a, size_t row, size_t col)
{
    size_t blk = col >> 8;
    int w = (int)(col & 255), grp = w >> 6, n = (w >> 5) & 1, l = w & 31;
    float d = f16_bits_to_f32(a.at(row, blk, 0), a.at(row, blk, 1));
    float dmin = f16_bits_to_f32(a.at(row, blk, 2), a.at(row, blk, 3));
    int j = 2 * grp + n;
    uint32_t sc, mn;
    if (j < 4) {
        sc = a.at(row, blk, 4 + j) & 63;
        mn = a.at(row, blk, 4 + j + 4) & 63;
    } else {
        uint32_t hi4 = a.at(row, blk, 4 + j + 4);
        sc = (hi4 & 0x0F) | ((a.at(row, blk, 4 + j - 4) >> 6) << 4);
        mn = (hi4 >> 4) | ((a.at(row, blk, 4 + j) >> 6) << 4);
    }
    uint32_t qb = a.at(row, blk, 48 + 32 * grp + l);
    uint32_t q = (n ? (qb >> 4) : (qb & 0x0F)) + (((a.at(row, blk, 16 + l) >> j) & 1u) ? 16u : 0u);
    float d1 = __fmul_rn(d, (float)sc), mm = __fmul_rn(dmin, (float)mn);
    return __fsub_rn(__fmul_rn(d1, (float)q), mm);
}

template <class Acc>
__device__ float deq_elem_q6k(const Acc& a, size_t row, size_t col)
{
    size_t blk = col >> 8;
    int w = (int)(col & 255), half = w >> 7, k = (w >> 5) & 3, l = w & 31, is = l >> 4;
    float d = f16_bits_to_f32(a.at(row, blk, 208), a.at(row, blk, 209));
    uint32_t qlb = a.at(row, blk, 64 * half + 32 * (k & 1) + l);
    uint32_t lo = (k & 2) ? (qlb >> 4) : (qlb & 0x0F);
    uint32_t hb = (a.at(row, blk, 128 + 32 * half + l) >> (2 * k)) & 3;
    int q = (int)(lo | (hb << 4)) - 32;
    int sc = (int)(int8_t)a.at(row, blk, 192 + 8 * half + is + 2 * k);
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
}

template <class Acc>
__device__ float deq_elem_q8_0(const Acc& a, size_t row, size_t col)
{
    size_t blk = col >> 5;
    int j = (int)(col & 31);
    float d = f16_bits_to_f32(a.at(row, blk, 0), a.at(row, blk, 1));
    return __fmul_rn((float)(int8_t)a.at(row, blk, 2 + j), d);
}

template <int TY, class Acc, bool BF16>
__global__ void dequant_kernel(Acc a, size_t rows, size_t cols, void* __restrict__ out)
{
    size_t total = rows * cols;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t row = i / cols, col = i % cols;
        float v = TY == kGgmlQ4K   ? deq_elem_q4k(a, row, col)
                  : TY == kGgmlQ5K ? deq_elem_q5k(a, row, col)
                  : TY == kGgmlQ6K ? deq_elem_q6k(a, row, col)
                                   : deq_elem_q8_0(a, row, col);
        if (BF16) reinterpret_cast<uint16_t*>(out)[i] = bf16_rne_bits(v);
        else reinterpret_cast<float*>(out)[i] = v;
    }
}

template <int TY, class Acc>
static void launch_deq(cudaStream_t st, Acc a, size_t rows, size_t cols, void* out, bool bf16)
{
    int grid = grid_for(rows * cols, 256);
    if (bf16) dequant_kernel<TY, Acc, true><<<grid, 256, 0, st>>>(a, rows, cols, out);
    else dequant_kernel<TY, Acc, false><<<grid, 256, 0, st>>>(a, rows, cols, out);
}

int32_t launch_dequant_weights(cudaStream_t st, uint32_t ty, const DeviceWeights& w, void* out, bool bf16)
{
    if (w.rows == 0 || w.cols == 0) return kOk;
    if (ty == kGgmlQ4K) launch_deq<kGgmlQ4K>(st, UnitQ4K{w.units, w.nblk, 0}, w.rows, w.cols, out, bf16);
    else if (ty == kGgmlQ5K) launch_deq<kGgmlQ5K>(st, UnitQ5K{w.units, w.nblk, 0}, w.rows, w.cols, out, bf16);
    else if (ty == kGgmlQ6K) launch_deq<kGgmlQ6K>(st, UnitQ6K{w.units, w.nblk, 0}, w.rows, w.cols, out, bf16);
    else launch_deq<kGgmlQ8_0>(st, PlanesQ8{w.q8_qs, w.q8_d, w.nblk, 0}, w.rows, w.cols, out, bf16);
    FERRIC_CUDA_TRY(cudaGetLastError());
    return kOk;
}

// n elements of one flat run of raw blocks (deq_raw): treated as a single row of n columns.
int32_t launch_dequant_raw(cudaStream_t st, uint32_t ty, const uint8_t* raw, size_t n, void* out, bool bf16)
{
    if (n == 0) return kOk;
    if (ty == kGgmlQ4K) launch_deq<kGgmlQ4K>(st, RawBytes{raw, n / 256, kQ4KBlock}, 1, n / 256 * 256, out, bf16);
    else if (ty == kGgmlQ5K) launch_deq<kGgmlQ5K>(st, RawBytes{raw, n / 256, kQ5KBlock}, 1, n / 256 * 256, out, bf16);
    else if (ty == kGgmlQ6K) launch_deq<kGgmlQ6K>(st, RawBytes{raw, n / 256, kQ6KBlock}, 1, n / 256 * 256, out, bf16);
    else launch_deq<kGgmlQ8_0>(st, RawBytes{raw, n / 32, kQ8Block}, 1, n / 32 * 32, out, bf16);
    FERRIC_CUDA_TRY(cudaGetLastError());
    return kOk;
}

}  // namespace ferric
