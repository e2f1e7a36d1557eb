// Batched decode product (M > 8; Q4_K and Q6_K) on the tcgen05 tensor cores with exact integer arithmetic.
//
// The mma.sync GEMV (kernels_gemv.cu) is bound by instruction issue beyond a few activation rows.  This
// kernel keeps its number format -- activations as four balanced base-128 limbs of X = rint(x * 2^(27-e)),
// one e per (activation row, super-block) -- and moves the multiply-accumulates to tcgen05.mma kind::f16 on
// INTEGER-VALUED f16 operands, which makes the tensor core an exact integer engine:
//   A[row][k] = sc(row, sub-block of k) * q(row, k)      0 .. 63 * 15 = 945        exact in f16
//   B[4b+j][k] = limb j of activation row b               -64 .. 63                 exact in f16
//   one super-block (K = 256) accumulates at most 256 * 945 * 64 < 2^24 in f32 -- every partial sum is an
//   integer the accumulator represents exactly, so neither rounding nor the order of the adds matters.
// After each super-block four drain warps read the accumulator back and apply what differs per row and
// super-block in f32: y[b][row] += 2^(e-6) * (d * V - dmin * sum_sb m_sb * S_sb), V = the limbs recombined,
// S_sb = the activation sums of the eight sub-blocks (from the preparation kernel).  The accumulator is
// double-buffered in tensor memory, so the drain of one super-block overlaps the MMAs of the next.
// This replaces, for M > 8, the same reference operator as the GEMV: Tensor::matmul_q4_k
// (crates/ferric-tensor/src/dtype.rs:1426-1473).
//
// CTA = 128 weight rows x N_TILE / 4 activation rows (N_TILE = 64, 128, 256 operand rows) x a range of
// super-blocks (K split across blockIdx.z for matrices with few row tiles; partials are summed in a fixed order
// by the finish kernel, which also applies the SwiGLU epilogue).
//   warp 0   weight producer (bulk copies of raw quant units)        warp 2      limb producer (TMA)
//   warp 1   MMA issuer, tensor-memory owner                         warps 3..10 operand makers (sc * q -> f16)
//   warps 11..14 drain
// Every mbarrier wait is bounded; a wait that runs out records a code that ferric_cuda_gemm_status reports.
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"
#include "layout.h"
#include "tc_common.cuh"

namespace ferric {

constexpr int kTcRows = 128;          // weight rows per CTA (UMMA M)
constexpr int kTcChunkK = 64;         // K per stage: 64 f16 = one 128-byte swizzle row
constexpr int kTcRawStages = 2;
constexpr int kTcMetaStages = 8;      // per-row (d, dmin, mins) of the super-blocks between the makers and the drain
constexpr int kTcMakerWarps = 8, kTcDrainWarps = 8;   // two drain warps per TMEM lane quarter, half the activation rows each
constexpr int kTcFirstMaker = 3, kTcFirstDrain = kTcFirstMaker + kTcMakerWarps;
constexpr int kTcThreads = 32 * (kTcFirstDrain + kTcDrainWarps);   // 608
constexpr int kTcABytes = kTcRows * 128;   // one operand plane of one K chunk
// Q4_K needs one operand plane (sc * q <= 945).  Q6_K's sc * (q - 32) reaches 127 * 32 = 4064, beyond the integers f16
// holds exactly, so its scale is split as sc = 16 sh + sl (sl 0..15, sh -8..7) into two planes sl * (q - 32) and
// sh * (q - 32), multiplied into two accumulators and recombined as D1 + 16 D2 in the drain.
__host__ __device__ constexpr int tc_planes(uint32_t ty) { return ty == kGgmlQ6K ? 2 : 1; }
__host__ __device__ constexpr int tc_unit_bytes(uint32_t ty) { return ty == kGgmlQ6K ? kQ6KUnit : kQ4KUnit; }
__host__ __device__ constexpr int tc_raw_bytes(uint32_t ty) { return 8 * tc_unit_bytes(ty); }
constexpr int kTcMaxBStages = 8;

struct TcRowMeta {
    float d, dmin;
    uint32_t m_lo, m_hi;   // the eight 6-bit mins, one per byte
};
static_assert(sizeof(TcRowMeta) == 16, "row meta is one 16-byte store");

constexpr int kTcSumFloats = 64 * 9;   // per stage: up to 64 activation rows x (8 sub-block sums + 1 scale)
__host__ __device__ constexpr int tc_a_stages(uint32_t ty, int) { return ty == kGgmlQ6K ? 3 : 4; }
__host__ __device__ constexpr int tc_fixed_bytes(uint32_t ty, int n_tile)
{
    return 1024 /*align*/ + 512 /*barriers*/ + tc_a_stages(ty, n_tile) * tc_planes(ty) * kTcABytes + kTcRawStages * tc_raw_bytes(ty) +
           kTcMetaStages * kTcRows * (int)sizeof(TcRowMeta) + 2 * kTcSumFloats * 4;
}
__host__ __device__ constexpr int tc_b_bytes(int n_tile) { return n_tile * 128; }
__host__ __device__ constexpr int tc_b_stages(uint32_t ty, int n_tile)
{
    return (232448 - tc_fixed_bytes(ty, n_tile)) / tc_b_bytes(n_tile) > kTcMaxBStages
               ? kTcMaxBStages
               : (232448 - tc_fixed_bytes(ty, n_tile)) / tc_b_bytes(n_tile);
}
__host__ __device__ constexpr int tc_smem_bytes(uint32_t ty, int n_tile)
{
    return tc_fixed_bytes(ty, n_tile) + tc_b_stages(ty, n_tile) * tc_b_bytes(n_tile);
}
static_assert(tc_b_stages(kGgmlQ4K, 256) >= 3 && tc_b_stages(kGgmlQ6K, 128) >= 3, "limb stages at the widest tiles");

struct TcBarriers {
    uint64_t raw_full[kTcRawStages], raw_empty[kTcRawStages];
    uint64_t a_full[4], a_empty[4];
    uint64_t b_full[kTcMaxBStages], b_empty[kTcMaxBStages];
    uint64_t acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    int abort;
};
static_assert(sizeof(TcBarriers) <= 512, "barrier block");

// kind::f16 with f16 operands (formats 0), f32 accumulator, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n)
{
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------------------------------------
// Activation preparation for this kernel: x (f32) -> limb matrix XL[4 * m][cols] (f16 integers, row 4b + j =
// limb j of activation row b), SS[nblk][m_pad][8] = sub-block sums of X scaled by 2^-21, UP[nblk][m_pad] = 2^(e-6)
// (super-block major, so that what one CTA needs for one super-block is contiguous).
// One warp per (pair of activation rows, super-block), lanes 0..15 row 0, lanes 16..31 row 1, 16 values each --
// the same scaling and limb split as the GEMV's preparation.
// ------------------------------------------------------------------------------------------
constexpr int kTcPrepWarps = 4;
__global__ void __launch_bounds__(32 * kTcPrepWarps)
tc_prep_kernel(const float* __restrict__ x, size_t m, size_t m_pad, size_t ldx, size_t nblk, __half* __restrict__ xl, size_t ldxl,
               float* __restrict__ ss, float* __restrict__ up)
{
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, prow = lane >> 4, q = lane & 15;
    const size_t pairs = (m + 1) / 2, wid = blockIdx.x * (size_t)kTcPrepWarps + warp;
    if (wid >= pairs * nblk) return;
    const size_t pair = wid / nblk, blk = wid % nblk, b = 2 * pair + (size_t)prow;
    const bool valid = b < m;
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = 0.0f;
    if (valid) {
        const float4* p = reinterpret_cast<const float4*>(x + b * ldx + blk * 256 + 16 * q);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 f = ld_act(p + i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    int e = 0;
    if (amax > 0.0f && amax < INFINITY) {
        (void)frexpf(amax, &e);
        e += 1;                  // 2^e >= 2 max|x|
        if (e < -80) e = -80;
        if (e > 120) e = 120;
    }
    const float to_int = ldexpf(1.0f, 27 - e);
    int sum = 0;
    uint32_t h[kLimbs][8];     // limb j of values 2i, 2i+1 as two f16 integers
#pragma unroll
    for (int i = 0; i < 16; i++) {
        int X = __float2int_rn(v[i] * to_int);
        sum += X;                // |X| <= 2^26, sixteen of them fit
        int a[kLimbs];
        a[3] = ((X + 64) & 127) - 64; X = (X - a[3]) >> 7;
        a[2] = ((X + 64) & 127) - 64; X = (X - a[2]) >> 7;
        a[1] = ((X + 64) & 127) - 64; X = (X - a[1]) >> 7;
        a[0] = X;
#pragma unroll
        for (int j = 0; j < kLimbs; j++) {
            const uint32_t bits = (uint32_t)__half_as_ushort(__int2half_rn(a[j]));
            if (i & 1) h[j][i >> 1] |= bits << 16;
            else h[j][i >> 1] = bits;
        }
    }
    if (valid) {
#pragma unroll
        for (int j = 0; j < kLimbs; j++) {
            uint4* dst = reinterpret_cast<uint4*>(xl + (4 * b + j) * ldxl + blk * 256 + 16 * q);
            dst[0] = make_uint4(h[j][0], h[j][1], h[j][2], h[j][3]);
            dst[1] = make_uint4(h[j][4], h[j][5], h[j][6], h[j][7]);
        }
    }
    // sub-block (32 values = two lanes) sums, scaled so that they combine with V (units of 2^-21 * 2^21)
    const float s16 = (float)sum * 4.76837158203125e-07f;   // 2^-21
    const float s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 1);
    if (valid && (q & 1) == 0) ss[(blk * m_pad + b) * 8 + (q >> 1)] = s32;
    if (valid && q == 0) up[blk * m_pad + b] = ldexpf(1.0f, e - 6);
}

// ------------------------------------------------------------------------------------------
// Eight weights (one 4-bit value in each byte of w0, w1, at bit `shift`) times the integer scale -> eight f16
// integers.  Two values per 32-bit multiply (products <= 945 stay inside their 16-bit lanes); 0x6400 | v is
// the f16 1024 + v, and subtracting 1024 is exact for v < 1024.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 tc_make8(uint32_t w0, uint32_t w1, int shift, uint32_t sc)
{
    const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
    auto four = [&](uint32_t w, uint32_t& lo, uint32_t& hi) {
        const uint32_t p02 = (((w >> shift) & 0x000F000Fu) * sc) | 0x64006400u;         // values 0, 2
        const uint32_t p13 = (((w >> (shift + 8)) & 0x000F000Fu) * sc) | 0x64006400u;   // values 1, 3
        const __half2 h02 = __hsub2(*reinterpret_cast<const __half2*>(&p02), k1024);
        const __half2 h13 = __hsub2(*reinterpret_cast<const __half2*>(&p13), k1024);
        const uint32_t u02 = *reinterpret_cast<const uint32_t*>(&h02), u13 = *reinterpret_cast<const uint32_t*>(&h13);
        lo = __byte_perm(u02, u13, 0x5410);   // values 0, 1
        hi = __byte_perm(u02, u13, 0x7632);   // values 2, 3
    };
    uint4 o;
    four(w0, o.x, o.y);
    four(w1, o.z, o.w);
    return o;
}

// ---------------------------------------------------------------- operand makers
// One call per maker warp.  Warp = one 16-row unit, lane = (row g / g+8, 8-byte piece t), with the prefill kernel's
// conflict-free lane map.  Returns 0 or the code of the wait that ran out.
template <int A_STAGES>
__device__ __forceinline__ int tc_make_q4k(TcBarriers* bar, uint8_t* a_stage, const uint8_t* raw_stage, TcRowMeta* meta, int nb,
                                           int tiles_here, int wd, int lane)
{
    constexpr int kTcAStages = A_STAGES;
    int fail = 0;
    // ---------------- operand makers: warp = one 16-row unit, lane = (row g / g+8, 8-byte piece t); see the
    // prefill kernel for the conflict-free lane map
    const int t = lane & 3, qd = lane >> 3, g = ((lane >> 2) & 1) ? (qd ^ 5) : qd;
    const bool unit_ok = wd < tiles_here;
    const uint32_t arow_off = (uint32_t)(2 * wd * 1024 + g * 128);
    const uint32_t col_lo = (uint32_t)((t ^ g) << 4), col_hi = (uint32_t)(((4 + t) ^ g) << 4);
    for (int i = 0; i < nb && !fail; i++) {
        const int rs = i % kTcRawStages;
        if (!mbar_wait(&bar->raw_full[rs], ((uint32_t)i / kTcRawStages) & 1u)) { fail = 4; break; }
        const uint8_t* u = raw_stage + rs * (8 * kQ4KUnit) + wd * kQ4KUnit;
        uint4 hdr[2], qs[2][2];
#pragma unroll
        for (int hi = 0; hi < 2; hi++) {
            hdr[hi] = qs[hi][0] = qs[hi][1] = make_uint4(0, 0, 0, 0);
            if (unit_ok) {
                hdr[hi] = *reinterpret_cast<const uint4*>(u + 16 * (g + 8 * hi));
                qs[hi][0] = *reinterpret_cast<const uint4*>(u + 256 + 512 * (2 * hi) + 16 * (4 * g + t));
                qs[hi][1] = *reinterpret_cast<const uint4*>(u + 256 + 512 * (2 * hi + 1) + 16 * (4 * g + t));
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar->raw_empty[rs]);
        if (t == 0) {   // hand (d, dmin, mins) of this super-block's rows to the drain
#pragma unroll
            for (int hi = 0; hi < 2; hi++) {
                uint32_t mn[8], sc_unused;
#pragma unroll
                for (int sb = 0; sb < 8; sb++) q4k_scale_min(hdr[hi], sb, sc_unused, mn[sb]);
                TcRowMeta rm;
                rm.d = __half2float(__ushort_as_half((unsigned short)(hdr[hi].x & 0xffffu)));
                rm.dmin = __half2float(__ushort_as_half((unsigned short)(hdr[hi].x >> 16)));
                rm.m_lo = mn[0] | (mn[1] << 8) | (mn[2] << 16) | (mn[3] << 24);
                rm.m_hi = mn[4] | (mn[5] << 8) | (mn[6] << 16) | (mn[7] << 24);
                *reinterpret_cast<uint4*>(&meta[(i % kTcMetaStages) * kTcRows + 16 * wd + 8 * hi + g]) =
                    *reinterpret_cast<const uint4*>(&rm);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint4 lo[2], up8[2];
#pragma unroll
            for (int hi = 0; hi < 2; hi++) {
                uint32_t sc0, sc1, mn_unused;
                q4k_scale_min(hdr[hi], 2 * j, sc0, mn_unused);
                q4k_scale_min(hdr[hi], 2 * j + 1, sc1, mn_unused);
                const uint4 q4 = qs[hi][j >> 1];
                const uint32_t w0 = (j & 1) ? q4.z : q4.x, w1 = (j & 1) ? q4.w : q4.y;
                lo[hi] = tc_make8(w0, w1, 0, sc0);
                up8[hi] = tc_make8(w0, w1, 4, sc1);
            }
            const int c = 4 * i + j, s = c % kTcAStages;
            // (every lane polls: one polling lane plus a shuffle was measured 15 % slower -- the wake-up is on the critical path)
            if (!mbar_wait(&bar->a_empty[s], (((uint32_t)c / kTcAStages) & 1u) ^ 1u)) { fail = 5; break; }
            uint8_t* arow = a_stage + s * kTcABytes + arow_off;
#pragma unroll
            for (int hi = 0; hi < 2; hi++) {
                *reinterpret_cast<uint4*>(arow + hi * 1024 + col_lo) = lo[hi];
                *reinterpret_cast<uint4*>(arow + hi * 1024 + col_hi) = up8[hi];
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->a_full[s]);   // also publishes this block's row meta (written above)
        }
    }
    return fail;
}

// Four Q6_K weights (6-bit values in the bytes of q) times one scale digit -> four f16 integers mult * (q - 32),
// negated when `neg`: two values per 32-bit multiply (q * mult <= 63 * 15), 0x6400 | v = 1024 + v in f16, and
// subtracting 1024 + 32 * mult (exact, <= 1504) leaves mult * (q - 32) exactly.
__device__ __forceinline__ uint2 tc_make4_q6(uint32_t q, uint32_t mult, bool neg)
{
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)(0x6400u + 32u * mult)));   // 1024 + 32 mult: exact bits
    const uint32_t p02 = ((q & 0x00FF00FFu) * mult) | 0x64006400u;          // values 0, 2
    const uint32_t p13 = (((q >> 8) & 0x00FF00FFu) * mult) | 0x64006400u;   // values 1, 3
    const __half2 h02 = __hsub2(*reinterpret_cast<const __half2*>(&p02), bias);
    const __half2 h13 = __hsub2(*reinterpret_cast<const __half2*>(&p13), bias);
    const uint32_t sign = neg ? 0x80008000u : 0u;
    const uint32_t u02 = *reinterpret_cast<const uint32_t*>(&h02) ^ sign, u13 = *reinterpret_cast<const uint32_t*>(&h13) ^ sign;
    return make_uint2(__byte_perm(u02, u13, 0x5410), __byte_perm(u02, u13, 0x7632));
}

// Q6_K (unit layout in layout.h; lane ownership as in the prefill kernel's Q6_K stage): two operand planes per chunk,
// plane 0 = sl * (q - 32), plane 1 = sh * (q - 32) with sc = 16 sh + sl.  Row meta carries d only.
template <int A_STAGES>
__device__ __forceinline__ int tc_make_q6k(TcBarriers* bar, uint8_t* a_stage, const uint8_t* raw_stage, TcRowMeta* meta, int nb,
                                           int tiles_here, int wd, int lane)
{
    constexpr int kStageBytes = 2 * kTcABytes;
    int fail = 0;
    const int t = lane & 3, qd = lane >> 3, g = ((lane >> 2) & 1) ? (qd ^ 5) : qd;
    const bool unit_ok = wd < tiles_here;
    const uint32_t arow_off = (uint32_t)(2 * wd * 1024 + g * 128);
    for (int i = 0; i < nb && !fail; i++) {
        const int rs = i % kTcRawStages;
        if (!mbar_wait(&bar->raw_full[rs], ((uint32_t)i / kTcRawStages) & 1u)) { fail = 4; break; }
        const uint8_t* u = raw_stage + rs * (8 * kQ6KUnit) + wd * kQ6KUnit;
        uint4 ql[2][2], qh[2], sc[2];
        uint32_t dpair = 0;
#pragma unroll
        for (int hi = 0; hi < 2; hi++) {
            ql[hi][0] = ql[hi][1] = qh[hi] = sc[hi] = make_uint4(0, 0, 0, 0);
            if (unit_ok) {
                ql[hi][0] = *reinterpret_cast<const uint4*>(u + kQ6KOffQl + 512 * (2 * hi) + 16 * (4 * g + t));
                ql[hi][1] = *reinterpret_cast<const uint4*>(u + kQ6KOffQl + 512 * (2 * hi + 1) + 16 * (4 * g + t));
                qh[hi] = *reinterpret_cast<const uint4*>(u + kQ6KOffQh + 512 * hi + 16 * (4 * g + t));
                sc[hi] = *reinterpret_cast<const uint4*>(u + kQ6KOffSc + 16 * (g + 8 * hi));
            }
        }
        if (unit_ok) dpair = *reinterpret_cast<const uint32_t*>(u + 4 * g);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar->raw_empty[rs]);
        if (t == 0) {
#pragma unroll
            for (int hi = 0; hi < 2; hi++) {
                TcRowMeta rm;
                rm.d = __half2float(__ushort_as_half((unsigned short)(hi ? (dpair >> 16) : (dpair & 0xffffu))));
                rm.dmin = 0.0f;
                rm.m_lo = rm.m_hi = 0u;
                *reinterpret_cast<uint4*>(&meta[(i % kTcMetaStages) * kTcRows + 16 * wd + 8 * hi + g]) = *reinterpret_cast<const uint4*>(&rm);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // chunk j = (h, kp): sub-blocks k = 2 kp + c (c = 0, 1), is = 0, 1; scale byte 4 j + 2 c + is of the row's 16
            const int h = j >> 1, kp = j & 1;
            uint2 p0[2][4], p1[2][4];
#pragma unroll
            for (int hi = 0; hi < 2; hi++) {
                const uint32_t scw = j == 0 ? sc[hi].x : (j == 1 ? sc[hi].y : (j == 2 ? sc[hi].z : sc[hi].w));
#pragma unroll
                for (int c = 0; c < 2; c++) {
#pragma unroll
                    for (int is = 0; is < 2; is++) {
                        const int scv = (int)(int8_t)(scw >> (8 * (2 * c + is)));
                        const int sl = scv & 15, sh = scv >> 4;           // scv = 16 sh + sl
                        const uint4 qlv = ql[hi][c];
                        const uint32_t lw = (2 * h + is) == 0 ? qlv.x : ((2 * h + is) == 1 ? qlv.y : ((2 * h + is) == 2 ? qlv.z : qlv.w));
                        const uint32_t hw = (2 * h + is) == 0 ? qh[hi].x : ((2 * h + is) == 1 ? qh[hi].y : ((2 * h + is) == 2 ? qh[hi].z : qh[hi].w));
                        const uint32_t q = ((lw >> (4 * kp)) & 0x0F0F0F0Fu) | (((hw >> (2 * (2 * kp + c))) & 0x03030303u) << 4);
                        p0[hi][2 * c + is] = tc_make4_q6(q, (uint32_t)sl, false);
                        p1[hi][2 * c + is] = tc_make4_q6(q, (uint32_t)(sh < 0 ? -sh : sh), sh < 0);
                    }
                }
            }
            const int c4 = 4 * i + j, s = c4 % A_STAGES;
            if (!mbar_wait(&bar->a_empty[s], (((uint32_t)c4 / A_STAGES) & 1u) ^ 1u)) { fail = 5; break; }
            uint8_t* arow = a_stage + s * kStageBytes + arow_off;
#pragma unroll
            for (int hi = 0; hi < 2; hi++)
#pragma unroll
                for (int k = 0; k < 4; k++) {   // k = 2c + is: 16-byte column 2k + (t >> 1), half t & 1
                    const uint32_t off = (uint32_t)(hi * 1024 + (((2 * k + (t >> 1)) ^ g) << 4) + 8 * (t & 1));
                    *reinterpret_cast<uint2*>(arow + off) = p0[hi][k];
                    *reinterpret_cast<uint2*>(arow + kTcABytes + off) = p1[hi][k];
                }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->a_full[s]);
        }
    }
    return fail;
}

template <uint32_t TY, int N_TILE>
__global__ void __launch_bounds__(kTcThreads, 1)
gemv_tc_kernel(const uint8_t* __restrict__ units, const __grid_constant__ CUtensorMap xmap, const float* __restrict__ ss,
                   const float* __restrict__ up, float* __restrict__ out, size_t ld_out, size_t split_stride, int rows, int nblk,
                   int m, int m_pad, int row_tiles16, int blocks_per_split, int* __restrict__ err)
{
    extern __shared__ uint8_t tc_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int kBStages = tc_b_stages(TY, N_TILE), kBBytes = tc_b_bytes(N_TILE), kActs = N_TILE / 4;
    constexpr int kTcAStages = tc_a_stages(TY, N_TILE), kPlanes = tc_planes(TY), kAStageBytes = kPlanes * kTcABytes;
    constexpr int kUnit = tc_unit_bytes(TY), kTcRawBytes = tc_raw_bytes(TY);
    uint8_t* a_stage = smem;                                  // [kTcAStages][kPlanes][16384]
    uint8_t* b_stage = a_stage + kTcAStages * kAStageBytes;
    uint8_t* raw_stage = b_stage + kBStages * kBBytes;
    TcRowMeta* meta = reinterpret_cast<TcRowMeta*>(raw_stage + kTcRawStages * kTcRawBytes);   // [kTcMetaStages][128]
    float* sums = reinterpret_cast<float*>(meta + kTcMetaStages * kTcRows);   // [2][kActs * 9]: staged SS and UP of a super-block
    TcBarriers* bar = reinterpret_cast<TcBarriers*>(sums + 2 * kTcSumFloats);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kTcRows, rt0 = blockIdx.x * 8, act0 = blockIdx.y * kActs;
    const int tiles_here = max(0, min(8, row_tiles16 - rt0));
    const int blk0 = blockIdx.z * blocks_per_split, nb = max(0, min(nblk, blk0 + blocks_per_split) - blk0);

    if (threadIdx.x == 0) {
        for (int i = 0; i < kTcRawStages; i++) {
            mbar_init(&bar->raw_full[i], 1);
            mbar_init(&bar->raw_empty[i], kTcMakerWarps);
        }
        for (int i = 0; i < kTcAStages; i++) {
            mbar_init(&bar->a_full[i], kTcMakerWarps);
            mbar_init(&bar->a_empty[i], 1);
        }
        for (int i = 0; i < kBStages; i++) {
            mbar_init(&bar->b_full[i], 1);
            mbar_init(&bar->b_empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&bar->acc_full[i], 1);
            mbar_init(&bar->acc_empty[i], kTcDrainWarps);
        }
        bar->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    constexpr int kTmemCols = 2 * kPlanes * N_TILE;   // two sets of accumulators (one per operand plane); a power of two >= 128
    static_assert(kTmemCols <= 512, "tensor memory holds 512 columns");
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_base)),
                     "n"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = bar->tmem_base;
    int fail = 0;

    if (warp == 0) {
        // ---------------- weight producer (weights are immutable: no need to wait for the previous kernel)
        if (lane == 0) {
            for (int i = 0; i < nb; i++) {
                const int rs = i % kTcRawStages;
                if (!mbar_wait(&bar->raw_empty[rs], (((uint32_t)i / kTcRawStages) & 1u) ^ 1u)) { fail = 1; break; }
                mbar_expect_tx(&bar->raw_full[rs], (uint32_t)(tiles_here * kUnit));
                for (int t = 0; t < tiles_here; t++)
                    bulk_g2s(raw_stage + rs * kTcRawBytes + t * kUnit, units + ((size_t)(rt0 + t) * nblk + blk0 + i) * kUnit, kUnit,
                             &bar->raw_full[rs]);
            }
        }
    } else if (warp == 2) {
        // ---------------- limb producer: [64 k x N_TILE operand rows] f16 per stage
        if (lane == 0) {
            pdl_wait();   // the limbs come from the preparation kernel launched just before
            for (int c = 0; c < 4 * nb; c++) {
                const int s = c % kBStages;
                if (!mbar_wait(&bar->b_empty[s], (((uint32_t)c / kBStages) & 1u) ^ 1u)) { fail = 2; break; }
                mbar_expect_tx(&bar->b_full[s], (uint32_t)kBBytes);
                tma_load_2d(b_stage + s * kBBytes, &xmap, (4 * blk0 + c) * kTcChunkK, 4 * act0, &bar->b_full[s]);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: four K chunks per super-block into accumulator set (i & 1).  This one thread's
        // instruction stream paces the kernel at narrow tiles, so it is kept lean: running stage counters instead of
        // modulo / division, barrier addresses and descriptor low words advanced by adds.
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(kTcRows, N_TILE);
            const uint32_t a_full0 = smem_u32(&bar->a_full[0]), a_empty0 = smem_u32(&bar->a_empty[0]);
            const uint32_t b_full0 = smem_u32(&bar->b_full[0]), b_empty0 = smem_u32(&bar->b_empty[0]);
            const uint32_t adesc0 = umma_desc_lo(smem_u32(a_stage)), bdesc0 = umma_desc_lo(smem_u32(b_stage));
            uint32_t sa = 0, pa = 0, sb = 0, pb = 0;     // stage and phase parity of the A and B rings
            for (int i = 0; i < nb && !fail; i++) {
                const int buf = i & 1;
                if (!mbar_wait(&bar->acc_empty[buf], (((uint32_t)i >> 1) & 1u) ^ 1u)) { fail = 3; break; }
                tc_fence_after();
                const uint32_t d0 = tmem_acc + (uint32_t)(buf * kPlanes * N_TILE);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (!mbar_try(a_full0 + 8 * sa, pa) && !mbar_wait(&bar->a_full[sa], pa)) { fail = 3; break; }
                    if (!mbar_try(b_full0 + 8 * sb, pb) && !mbar_wait(&bar->b_full[sb], pb)) { fail = 3; break; }
                    tc_fence_after();
                    const uint32_t ad = adesc0 + sa * (uint32_t)(kAStageBytes >> 4), bd = bdesc0 + sb * (uint32_t)(kBBytes >> 4);
#pragma unroll
                    for (int k4 = 0; k4 < 4; k4++)
#pragma unroll
                        for (int pl = 0; pl < kPlanes; pl++)
                            umma_f16_lo(d0 + pl * N_TILE, ad + (uint32_t)(pl * (kTcABytes >> 4) + 2 * k4), bd + 2 * k4, idesc,
                                        (j | k4) ? 1u : 0u);
                    umma_commit_addr(a_empty0 + 8 * sa);
                    umma_commit_addr(b_empty0 + 8 * sb);
                    if (++sa == (uint32_t)kTcAStages) { sa = 0; pa ^= 1u; }
                    if (++sb == (uint32_t)kBStages) { sb = 0; pb ^= 1u; }
                }
                if (!fail) umma_commit(&bar->acc_full[buf]);
            }
        }
    } else if (warp < kTcFirstDrain) {
        // ---------------- operand makers (per quant type, above)
        const int wd = warp - kTcFirstMaker;
        if (TY == kGgmlQ4K) fail = tc_make_q4k<kTcAStages>(bar, a_stage, raw_stage, meta, nb, tiles_here, wd, lane);
        else fail = tc_make_q6k<kTcAStages>(bar, a_stage, raw_stage, meta, nb, tiles_here, wd, lane);
    } else {
        // ---------------- drain: TMEM lane = weight row; column 4b + j = limb j of activation row act0 + b
        // two warps share a TMEM lane quarter; warp half h takes the groups of eight activation rows 2g + h
        const int q = warp & 3, rloc = 32 * q + lane, wrow = row0 + rloc, half = (warp - kTcFirstDrain) >> 2;
        constexpr int kGroups = kActs / 16;            // groups of eight activation rows per drain warp
        float acc[kGroups * 8];
#pragma unroll
        for (int b = 0; b < kGroups * 8; b++) acc[b] = 0.0f;
        pdl_wait();   // ss / up come from the preparation kernel
        // What the drain needs of a super-block besides the accumulator -- the activation rows' eight sub-block sums
        // and their scale -- is fetched one super-block ahead into registers and staged in shared memory.
        const int dt = threadIdx.x - 32 * kTcFirstDrain;          // 0..127
        auto fetch = [&](int i, float4& sv, float& uv) {
            sv = make_float4(0.f, 0.f, 0.f, 0.f);
            uv = 0.f;
            if (i < nb) {
                const size_t base = (size_t)(blk0 + i) * m_pad + act0;
                if (dt < kActs * 2) sv = __ldg(reinterpret_cast<const float4*>(ss + base * 8) + dt);
                if (dt < kActs) uv = __ldg(up + base + dt);
            }
        };
        auto stage = [&](int slot, const float4& sv, float uv) {
            float* dst = sums + slot * kTcSumFloats;
            if (dt < kActs * 2) reinterpret_cast<float4*>(dst)[dt] = sv;
            if (dt < kActs) dst[kActs * 8 + dt] = uv;
        };
        float4 sv;
        float uv;
        fetch(0, sv, uv);
        stage(0, sv, uv);
        named_bar_sync(1, 32 * kTcDrainWarps);
        for (int i = 0; i < nb && !fail; i++) {
            const int buf = i & 1;
            fetch(i + 1, sv, uv);
            if (!mbar_wait(&bar->acc_full[buf], ((uint32_t)i >> 1) & 1u)) { fail = 6; break; }
            tc_fence_after();
            const TcRowMeta rm = meta[(i % kTcMetaStages) * kTcRows + rloc];
            const float* sl = sums + (i & 1) * kTcSumFloats;
            float mf[8];
#pragma unroll
            for (int sb = 0; sb < 4; sb++) {
                mf[sb] = (float)((rm.m_lo >> (8 * sb)) & 0xffu);
                mf[4 + sb] = (float)((rm.m_hi >> (8 * sb)) & 0xffu);
            }
#pragma unroll
            for (int gg = 0; gg < kGroups; gg++) {
                const int grp = 2 * gg + half;
                uint32_t v[32];
                tmem_ld_32(tmem_acc + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * kPlanes * N_TILE + 32 * grp), v);
                if (kPlanes == 2) {   // second scale digit: D1 + 16 D2
                    uint32_t w[32];
                    tmem_ld_32(tmem_acc + ((uint32_t)(32 * q) << 16) + (uint32_t)((buf * kPlanes + 1) * N_TILE + 32 * grp), w);
#pragma unroll
                    for (int e = 0; e < 32; e++) v[e] = __float_as_uint(fmaf(16.0f, __uint_as_float(w[e]), __uint_as_float(v[e])));
                }
#pragma unroll
                for (int bb = 0; bb < 8; bb++) {
                    const int b = 8 * grp + bb;
                    const float scale = sl[kActs * 8 + b];
                    float V = __uint_as_float(v[4 * bb + 3]);
                    V = fmaf(V, 0.0078125f, __uint_as_float(v[4 * bb + 2]));
                    V = fmaf(V, 0.0078125f, __uint_as_float(v[4 * bb + 1]));
                    V = fmaf(V, 0.0078125f, __uint_as_float(v[4 * bb]));
                    if (TY == kGgmlQ4K) {
                        const float4 s0 = reinterpret_cast<const float4*>(sl)[2 * b], s1 = reinterpret_cast<const float4*>(sl)[2 * b + 1];
                        float Mn = mf[0] * s0.x;
                        Mn = fmaf(mf[1], s0.y, Mn); Mn = fmaf(mf[2], s0.z, Mn); Mn = fmaf(mf[3], s0.w, Mn);
                        Mn = fmaf(mf[4], s1.x, Mn); Mn = fmaf(mf[5], s1.y, Mn); Mn = fmaf(mf[6], s1.z, Mn); Mn = fmaf(mf[7], s1.w, Mn);
                        acc[8 * gg + bb] = fmaf(scale, fmaf(rm.d, V, -rm.dmin * Mn), acc[8 * gg + bb]);
                    } else {
                        acc[8 * gg + bb] = fmaf(scale * rm.d, V, acc[8 * gg + bb]);
                    }
                }
            }
            // every drain thread has finished reading the other slot (it did so one iteration ago and has met the
            // barrier below since), so the next super-block's values can go there
            stage((i + 1) & 1, sv, uv);
            named_bar_sync(1, 32 * kTcDrainWarps);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->acc_empty[buf]);
        }
        if (!fail && wrow < rows) {
            float* o = out + (size_t)blockIdx.z * split_stride;
#pragma unroll
            for (int gg = 0; gg < kGroups; gg++)
#pragma unroll
                for (int bb = 0; bb < 8; bb++) {
                    const int act = act0 + 8 * (2 * gg + half) + bb;
                    if (act < m) o[(size_t)act * ld_out + wrow] = acc[8 * gg + bb];
                }
        }
    }
    if (fail) {
        atomicExch(&bar->abort, fail);
        if (err) atomicExch(err, 16 + fail);
    }
    tc_fence_before();
    __syncthreads();
    if (bar->abort) {
        for (int i = 0; i < 200; i++) __nanosleep(1000);   // let copies still in flight land
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "n"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// Finish: y[b][r] = sum over K splits (in split order) of part[s][b][r]; with the SwiGLU epilogue the matrix is
// [gate rows | up rows] and y[b][o] = silu(gate) * up.
// ------------------------------------------------------------------------------------------
__global__ void tc_finish_kernel(const float* __restrict__ part, int splits, size_t split_stride, int m, int rows,
                                 float* __restrict__ y, size_t ldy, int swiglu)
{
    pdl_launch_dependents();
    pdl_wait();
    const int out_cols = swiglu ? rows / 2 : rows;
    const size_t total = (size_t)m * out_cols;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t b = idx / out_cols, o = idx % out_cols;
        float g = 0.0f, u = 0.0f;
        for (int s = 0; s < splits; s++) {
            const float* p = part + s * split_stride + b * (size_t)rows;
            g += p[o];
            if (swiglu) u += p[o + out_cols];
        }
        y[b * ldy + o] = swiglu ? silu_mul(g, u) : g;
    }
}

// ---------------------------------------------------------------- host side
int* gemm_status_word();   // device address of the status word shared with the prefill kernel (kernels_gemm.cu)

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn tc_encode_fn()
{
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct TcPlan {
    int n_tile, splits, blocks_per_split;
    size_t m_pad;                              // activation rows rounded up to whole tiles
    size_t off_ss, off_up, off_part, total;   // scratch offsets (XL at 0)
    bool needs_finish;
};

TcPlan tc_plan(uint32_t ty, const DeviceWeights& w, size_t m, Epilogue epi, int sm_count)
{
    TcPlan p;
    p.n_tile = m <= 16 ? 64 : ((m <= 32 || ty == kGgmlQ6K) ? 128 : 256);   // Q6_K: two accumulator planes, so half the width
    const size_t row_tiles = (w.rows + kTcRows - 1) / kTcRows, act_tiles = (4 * m + p.n_tile - 1) / p.n_tile;
    const size_t tiles = row_tiles * act_tiles;
    size_t splits = 1;
    if (tiles * 5 < (size_t)sm_count * 4) splits = ((size_t)sm_count + tiles - 1) / tiles;   // fill the machine along K
    if (splits > w.nblk) splits = w.nblk;
    if (splits > 16) splits = 16;
    p.blocks_per_split = (int)((w.nblk + splits - 1) / splits);
    p.splits = (int)((w.nblk + p.blocks_per_split - 1) / p.blocks_per_split);
    p.needs_finish = p.splits > 1 || epi == kEpiSwiglu;
    p.m_pad = act_tiles * (size_t)(p.n_tile / 4);
    p.off_ss = align256(4 * m * w.cols * sizeof(__half));
    p.off_up = p.off_ss + align256(p.m_pad * w.nblk * 8 * sizeof(float));
    p.off_part = p.off_up + align256(p.m_pad * w.nblk * sizeof(float));
    p.total = p.off_part + (p.needs_finish ? align256((size_t)p.splits * m * w.rows * sizeof(float)) : 0);
    return p;
}

template <uint32_t TY, int N_TILE>
int32_t launch_tc_tile(cudaStream_t st, const DeviceWeights& w, const CUtensorMap& map, const float* ss, const float* up, float* out,
                       size_t ld_out, size_t split_stride, size_t m, const TcPlan& p, bool pdl)
{
    static bool attr_done[64] = {};
    int dev = 0;
    FERRIC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !attr_done[dev]) {
        FERRIC_CUDA_TRY(cudaFuncSetAttribute(gemv_tc_kernel<TY, N_TILE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             tc_smem_bytes(TY, N_TILE)));
        attr_done[dev] = true;
    }
    dim3 grid((unsigned)((w.rows + kTcRows - 1) / kTcRows), (unsigned)((4 * m + N_TILE - 1) / N_TILE), (unsigned)p.splits);
    FERRIC_CUDA_TRY(launch_kernel(gemv_tc_kernel<TY, N_TILE>, grid, dim3(kTcThreads), (size_t)tc_smem_bytes(TY, N_TILE), st, pdl,
                                  (const uint8_t*)w.units, map, ss, up, out, ld_out, split_stride, (int)w.rows, (int)w.nblk,
                                  (int)m, (int)p.m_pad, (int)w.row_tiles(), p.blocks_per_split, gemm_status_word()));
    return kOk;
}
}  // namespace

bool gemv_tc_eligible(uint32_t ty, const DeviceWeights& w, size_t m)
{
    // Measured cross-over with the mma.sync GEMV (which runs in passes of 4 activation rows; 64-layer step at 12 / 16 / 24
    // rows: 12.4 / 15.3 / 21.0 ms in passes against 14.5 / 15.5 / 19.9 ms here): Q4_K from 17 rows, Q6_K -- two operand
    // planes, so twice the MMAs -- from 24.  FERRIC_CUDA_GEMV_TC_MIN_M overrides both; 0 disables the path.
    const char* env = getenv("FERRIC_CUDA_GEMV_TC_MIN_M");   // read per call: tests move the threshold
    const int forced = env ? atoi(env) : -1;
    if (ty != kGgmlQ4K && ty != kGgmlQ6K) return false;
    const int min_m = forced >= 0 ? forced : (ty == kGgmlQ4K ? 17 : 24);
    return min_m > 0 && m >= (size_t)min_m && m <= 4096 && w.nblk > 0 && w.rows > 0 && w.rows <= (size_t)INT32_MAX / 2;
}

size_t gemv_tc_scratch_bytes(uint32_t ty, const DeviceWeights& w, size_t m, Epilogue epi, int sm_count)
{
    return tc_plan(ty, w, m, epi, sm_count).total;
}

int32_t launch_gemv_tc(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const float* x, size_t m, size_t ldx, float* y, size_t ldy,
                       Epilogue epi, void* scratch, const GemvTuning& tune, int* launches)
{
    EncodeTiledFn enc = tc_encode_fn();
    if (!enc) {
        set_last_error("the CUDA driver does not export cuTensorMapEncodeTiled");
        return kErrCuda;
    }
    const TcPlan p = tc_plan(ty, w, m, epi, tune.sm_count);
    uint8_t* base = reinterpret_cast<uint8_t*>(scratch);
    __half* xl = reinterpret_cast<__half*>(base);
    float* ss = reinterpret_cast<float*>(base + p.off_ss);
    float* up = reinterpret_cast<float*>(base + p.off_up);
    float* part = reinterpret_cast<float*>(base + p.off_part);

    const size_t pairs = (m + 1) / 2, warps = pairs * w.nblk;
    FERRIC_CUDA_TRY(launch_kernel(tc_prep_kernel, dim3((unsigned)((warps + kTcPrepWarps - 1) / kTcPrepWarps)), dim3(32 * kTcPrepWarps),
                                  0, st, tune.pdl, x, m, p.m_pad, ldx, w.nblk, xl, w.cols, ss, up));
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)w.cols, (cuuint64_t)(4 * m)};
    const cuuint64_t strides[1] = {(cuuint64_t)w.cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTcChunkK, (cuuint32_t)p.n_tile};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xl, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled (limbs) failed with code %d", (int)r);
        return kErrCuda;
    }
    float* out = p.needs_finish ? part : y;
    const size_t ld_out = p.needs_finish ? w.rows : ldy, split_stride = m * w.rows;
    int32_t rc;
    if (ty == kGgmlQ6K) {
        if (p.n_tile == 64) rc = launch_tc_tile<kGgmlQ6K, 64>(st, w, map, ss, up, out, ld_out, split_stride, m, p, tune.pdl);
        else rc = launch_tc_tile<kGgmlQ6K, 128>(st, w, map, ss, up, out, ld_out, split_stride, m, p, tune.pdl);
    } else {
        if (p.n_tile == 64) rc = launch_tc_tile<kGgmlQ4K, 64>(st, w, map, ss, up, out, ld_out, split_stride, m, p, tune.pdl);
        else if (p.n_tile == 128) rc = launch_tc_tile<kGgmlQ4K, 128>(st, w, map, ss, up, out, ld_out, split_stride, m, p, tune.pdl);
        else rc = launch_tc_tile<kGgmlQ4K, 256>(st, w, map, ss, up, out, ld_out, split_stride, m, p, tune.pdl);
    }
    if (rc != kOk) return rc;
    *launches += 2;
    if (p.needs_finish) {
        const size_t total = m * (epi == kEpiSwiglu ? w.rows / 2 : w.rows);
        unsigned blocks = (unsigned)((total + 255) / 256);
        if (blocks > 4u * (unsigned)tune.sm_count) blocks = 4u * (unsigned)tune.sm_count;
        FERRIC_CUDA_TRY(launch_kernel(tc_finish_kernel, dim3(blocks), dim3(256), 0, st, tune.pdl, (const float*)part, p.splits,
                                      split_stride, (int)m, (int)w.rows, y, ldy, epi == kEpiSwiglu ? 1 : 0));
        *launches += 1;
    }
    return kOk;
}

}  // namespace ferric
