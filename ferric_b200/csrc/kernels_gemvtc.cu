// Batched decode product (M > 8; Q4_K, Q5_K and Q6_K) on the tcgen05 tensor cores with integer-valued f16 operands.
//
// The mma.sync GEMV (kernels_gemv.cu) is bound by instruction issue beyond a few activation rows.  This kernel
// moves the multiply-accumulates to tcgen05.mma kind::f16 and keeps every operand an integer that f16 holds exactly:
//   A[row][k]     = sc(row, sub-block of k) * q(row, k)     0 .. 63 * 15 = 945 (Q5_K: 63 * 31 = 1953)
//   B[2b + j][k]  = limb j of activation row b: X = rint(x * 2^(22-e)) = 2048 hi + lo, |hi| <= 1024, |lo| <= 1024,
//                   one e per (activation row, super-block)
// so every product is exact and the f32 accumulator (one super-block, K = 256, per pass) rounds only where a running
// sum passes 2^24, i.e. by 2^-24 of that sum: the precision of an f32 product of the exact weights with X.  X keeps
// 21 bits below the super-block's largest activation.
// The Q4_K / Q5_K min term rides the tensor core too: one more K = 16 step per super-block multiplies the rows' eight 6-bit
// mins (twice) with the two pieces of each limb's sub-block sums (from the preparation kernel) into a second
// accumulator.  After each super-block the drain warps read both accumulators back and apply what differs per row
// and super-block in f32: y[b][row] += 2^(e-11) * (d * V - dmin * Mn), V and Mn recombined from their two limb
// columns.  The accumulators are double-buffered in tensor memory, so the drain of one super-block overlaps the MMAs
// of the next.
// This replaces, for M > 8, the same reference operator as the GEMV: Tensor::matmul_q4_k
// (crates/ferric-tensor/src/dtype.rs:1426-1473).
//
// CTA = 128 weight rows x N_TILE / 2 activation rows (N_TILE = 64 or 128 operand rows) x a range of super-blocks
// (K split across blockIdx.z for matrices with few row tiles; partials are summed in a fixed order by the finish
// kernel, which also applies the SwiGLU epilogue).
//   warp 0   weight producer (bulk copies of raw quant units)        warp 2      limb producer (TMA)
//   warp 1   MMA issuer, tensor-memory owner                         warps 3..10 operand makers (sc * q -> f16)
//   warps 11..18 drain
// Every mbarrier wait is bounded; a wait that runs out records a code that ferric_cuda_gemm_status reports.
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"
#include "layout.h"
#include "tc_common.cuh"
#include "tpwide.cuh"

namespace ferric {

constexpr int kTcRows = 128;          // weight rows per CTA (UMMA M)
constexpr int kTcLimbs = 2;           // operand rows per activation row
// Operand order along K: within every aligned group of four positions the values sit as 0, 2, 1, 3 (what the operand
// makers produce without a byte shuffle); tc_kpos(i) = the position of value i.
__host__ __device__ constexpr int tc_kpos(int i) { return (i & ~3) | ((i & 1) << 1) | ((i >> 1) & 1); }
constexpr int kTcChunkK = 64;         // K per stage: 64 f16 = one 128-byte swizzle row
constexpr int kTcMaxRawStages = 2;
// Raw quant stages: two, except for Q6_K at the wide tile, where one leaves room for two K chunks per ring stage.  The makers
// copy a raw super-block into registers before they convert any of it, so its successor is in flight while they work.
__host__ __device__ constexpr int tc_raw_stages(uint32_t ty, int n_tile) { return (ty == kGgmlQ6K && n_tile > 64) ? 1 : 2; }
// Per-row (d, dmin) of the super-blocks between the makers and the drain: the makers run at most one super-block of ring
// plus the accumulator sets ahead of the drain -- 1 + 2 at the wide tile, 1 + 4 at the narrow one.
__host__ __device__ constexpr int tc_meta_stages(int n_tile) { return n_tile > 64 ? 4 : 8; }
constexpr int kTcMakerWarps = 8, kTcDrainWarps = 8;   // two drain warps per TMEM lane quarter, half the activation rows each
constexpr int kTcFirstMaker = 3, kTcFirstDrain = kTcFirstMaker + kTcMakerWarps;
constexpr int kTcThreads = 32 * (kTcFirstDrain + kTcDrainWarps);   // 608
constexpr int kTcABytes = kTcRows * 128;   // one operand plane of one K chunk
// Q4_K needs one operand plane (sc * q <= 945).  Q6_K's sc * (q - 32) reaches 127 * 32 = 4064, beyond the integers f16
// holds exactly, so its scale is split as sc = 16 sh + sl (sl 0..15, sh -8..7) into two planes sl * (q - 32) and
// sh * (q - 32), multiplied into two accumulators and recombined as D1 + 16 D2 in the drain.
__host__ __device__ constexpr int tc_planes(uint32_t ty) { return ty == kGgmlQ6K ? 2 : 1; }
__host__ __device__ constexpr int tc_unit_bytes(uint32_t ty) { return ty == kGgmlQ6K ? kQ6KUnit : ty == kGgmlQ5K ? kQ5KUnit : kQ4KUnit; }
// Q4_K and Q5_K (the same block with a fifth bit per weight: sc * q <= 63 * 31 = 1953, still an integer f16 holds) have mins
__host__ __device__ constexpr bool tc_has_mins(uint32_t ty) { return ty == kGgmlQ4K || ty == kGgmlQ5K; }
__host__ __device__ constexpr int tc_raw_bytes(uint32_t ty) { return 8 * tc_unit_bytes(ty); }
constexpr int kTcMaxStages = 8;

struct TcRowMeta {
    float d, dmin;
};
static_assert(sizeof(TcRowMeta) == 8, "row meta is one 8-byte store");
// The Q4_K / Q5_K min step has its own operand tiles outside the ring, both in the swizzled 128-byte-row layout of which a K = 16
// step reads 32 bytes per row: A2 (128 rows; slot i & 3 of its four 32-byte columns holds super-block i's mins) and B2
// (n_tile rows; slot i mod the number of accumulator sets).
__host__ __device__ constexpr int tc_min_bytes(uint32_t ty, int n_tile) { return tc_has_mins(ty) ? kTcABytes + n_tile * 128 : 0; }

constexpr int kTcSumFloats = 64;   // per stage: the scales 2^(e-11) of up to 64 activation rows
// One ring for both operands: a stage holds the A planes of one K chunk (made by the maker warps) and its B tile (the
// limbs, by TMA), filled under ONE barrier (eight maker arrivals + the producer's expect-tx) and released by ONE
// tcgen05.commit -- the MMA thread's waits and commits are what paces this kernel.
__host__ __device__ constexpr int tc_b_bytes(int n_tile) { return n_tile * 128; }
// K chunks per ring stage: two (half as many hand-overs than one)
__host__ __device__ constexpr int tc_chunks(uint32_t, int) { return 2; }
__host__ __device__ constexpr int tc_stage_bytes(uint32_t ty, int n_tile)
{
    return tc_chunks(ty, n_tile) * (tc_planes(ty) * kTcABytes + tc_b_bytes(n_tile));
}
__host__ __device__ constexpr int tc_fixed_bytes(uint32_t ty, int n_tile)
{
    return 1024 /*align*/ + 512 /*barriers*/ + tc_min_bytes(ty, n_tile) + tc_raw_stages(ty, n_tile) * tc_raw_bytes(ty) +
           tc_meta_stages(n_tile) * kTcRows * (int)sizeof(TcRowMeta) + 2 * kTcSumFloats * 4;
}
__host__ __device__ constexpr int tc_stages(uint32_t ty, int n_tile)
{
    return (232448 - tc_fixed_bytes(ty, n_tile)) / tc_stage_bytes(ty, n_tile) > kTcMaxStages
               ? kTcMaxStages
               : (232448 - tc_fixed_bytes(ty, n_tile)) / tc_stage_bytes(ty, n_tile);
}
__host__ __device__ constexpr int tc_smem_bytes(uint32_t ty, int n_tile)
{
    return tc_fixed_bytes(ty, n_tile) + tc_stages(ty, n_tile) * tc_stage_bytes(ty, n_tile);
}
// A row-meta slot of super-block j - META is rewritten by the makers at the start of super-block j.  By then they hold the
// ring stages of j - 1, so the MMAs of super-block j - 1 - R have completed (R = the ring's depth in super-blocks), which
// started only after the drain of j - 1 - R - A had handed its accumulator set back (A sets): META >= 1 + R + A.
__host__ __device__ constexpr bool tc_meta_ok(uint32_t ty, int n_tile)
{
    return tc_meta_stages(n_tile) >= 1 + (tc_stages(ty, n_tile) * tc_chunks(ty, n_tile) + 3) / 4 + 256 / n_tile;
}
static_assert(tc_meta_ok(kGgmlQ4K, 64) && tc_meta_ok(kGgmlQ4K, 128) && tc_meta_ok(kGgmlQ5K, 64) && tc_meta_ok(kGgmlQ5K, 128) &&
                  tc_meta_ok(kGgmlQ6K, 64) && tc_meta_ok(kGgmlQ6K, 128),
              "row-meta ring depth");
// The same count for the min step's A2 slots (four, slot i & 3 rewritten at the start of super-block i): the min MMA of
// super-block i - 4 must be over, i.e. i - 4 <= i - 1 - R.
static_assert((tc_stages(kGgmlQ4K, 64) * tc_chunks(kGgmlQ4K, 64) + 3) / 4 <= 3 && (tc_stages(kGgmlQ5K, 64) * tc_chunks(kGgmlQ5K, 64) + 3) / 4 <= 3 &&
                  (tc_stages(kGgmlQ4K, 128) * tc_chunks(kGgmlQ4K, 128) + 3) / 4 <= 3,
              "A2 slot ring depth");
static_assert(tc_stages(kGgmlQ4K, 128) >= 2 && tc_stages(kGgmlQ4K, 64) >= 2 && tc_stages(kGgmlQ5K, 128) >= 2 && tc_stages(kGgmlQ5K, 64) >= 2 &&
                  tc_stages(kGgmlQ6K, 128) >= 2 && tc_stages(kGgmlQ6K, 64) >= 2,
              "ring depth");

struct TcBarriers {
    uint64_t raw_full[kTcMaxRawStages], raw_empty[kTcMaxRawStages];
    uint64_t full[kTcMaxStages], empty[kTcMaxStages];
    uint64_t acc_full[4], acc_empty[4];
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
// Activation preparation for this kernel: x (f32) -> X = rint(x * 2^(22-e)), one e per (activation row, super-block)
// with 2^e > 2 max|x|, so |X| < 2^21, split as X = 2048 hi + lo (lo in [-1024, 1023], |hi| <= 1024: both integers
// f16 holds exactly).  Outputs:
//   XL[2 * m][cols]        f16, row 2b = hi, row 2b + 1 = lo of activation row b, in the operand order tc_kpos
//   SB[nblk][2 * m_pad][16] f16 (Q4_K, Q5_K): what the tensor core needs for the min term -- per super-block 16 values
//                          per operand row, [sb] and [8 + sb] = the two pieces (|piece| <= 128, and a multiple of 256
//                          up to 2^15: both exact) of the sum of that row's limb over sub-block sb
//   UP[nblk][m_pad]        2^(e-11): V = D_hi + 2^-11 D_lo times UP is the product in x's units
// One warp per (pair of activation rows, super-block), lanes 0..15 row 0, lanes 16..31 row 1, 16 values each.
// ------------------------------------------------------------------------------------------
constexpr int kTcPrepWarps = 4;
__global__ void __launch_bounds__(32 * kTcPrepWarps)
tc_prep_kernel(const float* __restrict__ x, size_t m, size_t m_pad, size_t ldx, size_t nblk, __half* __restrict__ xl, size_t ldxl,
               __half* __restrict__ sb, float* __restrict__ up)
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
        e += 1;                  // 2^e > 2 max|x|
        if (e < -80) e = -80;
        if (e > 120) e = 120;
    }
    const float to_int = ldexpf(1.0f, 22 - e);
    int sum_hi = 0, sum_lo = 0;
    uint32_t h[kTcLimbs][8];     // limb j of values 2i, 2i+1 as two f16 integers
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const int X = __float2int_rn(v[i] * to_int);
        const int lo = ((X + 1024) & 2047) - 1024, hi = (X - lo) >> 11;
        sum_hi += hi;
        sum_lo += lo;
        const uint32_t bh = (uint32_t)__half_as_ushort(__int2half_rn(hi)), bl = (uint32_t)__half_as_ushort(__int2half_rn(lo));
        const int pos = tc_kpos(i);
        if (pos & 1) {
            h[0][pos >> 1] |= bh << 16;
            h[1][pos >> 1] |= bl << 16;
        } else {
            h[0][pos >> 1] = bh;
            h[1][pos >> 1] = bl;
        }
    }
    if (valid) {
#pragma unroll
        for (int j = 0; j < kTcLimbs; j++) {
            uint4* dst = reinterpret_cast<uint4*>(xl + (kTcLimbs * b + j) * ldxl + blk * 256 + 16 * q);
            dst[0] = make_uint4(h[j][0], h[j][1], h[j][2], h[j][3]);
            dst[1] = make_uint4(h[j][4], h[j][5], h[j][6], h[j][7]);
        }
    }
    // sub-block (32 values = two lanes) sums of each limb, in two exact pieces
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    if (sb != nullptr && valid && (q & 1) == 0) {
#pragma unroll
        for (int j = 0; j < kTcLimbs; j++) {
            const int s = j ? sum_lo : sum_hi, low = ((s + 128) & 255) - 128;
            __half* dst = sb + ((blk * m_pad + b) * kTcLimbs + j) * 16 + (q >> 1);
            dst[0] = __int2half_rn(low);
            dst[8] = __int2half_rn(s - low);
        }
    }
    if (valid && q == 0) up[blk * m_pad + b] = ldexpf(1.0f, e - 11);
}

// ------------------------------------------------------------------------------------------
// Operand making.  A small integer v sitting in a mantissa field of an f16 bit pattern is an exact number: bits 0..9
// under exponent pattern 0x6400 read 1024 + v, bits 4..7 under 0x5400 read 64 + v.  One half-precision fused
// multiply-add per PAIR of weights then gives scale * v exactly: (1024 + v) * sc - 1024 sc (the product is exact
// inside the FMA, the bias 1024 sc <= 64512 and the result <= 945 are f16 numbers).  A 32-bit word holds four weights,
// one per byte; bytes 0 and 2 form one pair, bytes 1 and 3 (after one shift) the other, and the pairs are stored as
// they come: within every aligned group of four K positions the operand order is 0, 2, 1, 3, and the preparation
// kernel stores the activation limbs in that same order.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ __half2 tc_h2(uint32_t u) { return *reinterpret_cast<const __half2*>(&u); }
__device__ __forceinline__ uint32_t tc_u32(__half2 h) { return *reinterpret_cast<const uint32_t*>(&h); }

// (1024 + b, 1024 + b) for byte `idx` (0..3) of `bytes`: one byte permute against the exponent byte 0x64
__device__ __forceinline__ __half2 tc_bcast_byte(uint32_t bytes, int idx)
{
    return tc_h2(__byte_perm(bytes, 0x64u, 0x4040u | (uint32_t)idx | ((uint32_t)idx << 8)));
}

// Sixteen Q4_K weights -- the low nibbles (sub-block 2j, scale sc_lo) and the high nibbles (sub-block 2j + 1, scale
// sc_hi) of the eight bytes of w0, w1 -- as f16 integers sc * q.  bias_lo = -1024 sc_lo, bias_hi = -64 sc_hi.
__device__ __forceinline__ void tc_make16(uint32_t w0, uint32_t w1, __half2 sc_lo, __half2 bias_lo, __half2 sc_hi, __half2 bias_hi,
                                          uint4& lo, uint4& hi)
{
    auto word = [&](uint32_t w, uint32_t& l02, uint32_t& l13, uint32_t& h02, uint32_t& h13) {
        const uint32_t t = w >> 8;
        l02 = tc_u32(__hfma2(tc_h2((w & 0x000F000Fu) | 0x64006400u), sc_lo, bias_lo));
        l13 = tc_u32(__hfma2(tc_h2((t & 0x000F000Fu) | 0x64006400u), sc_lo, bias_lo));
        h02 = tc_u32(__hfma2(tc_h2((w & 0x00F000F0u) | 0x54005400u), sc_hi, bias_hi));
        h13 = tc_u32(__hfma2(tc_h2((t & 0x00F000F0u) | 0x54005400u), sc_hi, bias_hi));
    };
    word(w0, lo.x, lo.y, hi.x, hi.y);
    word(w1, lo.z, lo.w, hi.z, hi.w);
}

// Eight weights given as one value per byte of b0, b1 (Q5_K: up to 31) -> f16 integers sc * v, bias = -1024 sc.
__device__ __forceinline__ uint4 tc_make8_bytes(uint32_t b0, uint32_t b1, __half2 sc, __half2 bias)
{
    uint4 o;
    o.x = tc_u32(__hfma2(tc_h2((b0 & 0x00FF00FFu) | 0x64006400u), sc, bias));
    o.y = tc_u32(__hfma2(tc_h2(((b0 >> 8) & 0x00FF00FFu) | 0x64006400u), sc, bias));
    o.z = tc_u32(__hfma2(tc_h2((b1 & 0x00FF00FFu) | 0x64006400u), sc, bias));
    o.w = tc_u32(__hfma2(tc_h2(((b1 >> 8) & 0x00FF00FFu) | 0x64006400u), sc, bias));
    return o;
}

// ---------------------------------------------------------------- operand makers
// One call per maker warp.  Warp = one 16-row unit, lane = (row g / g+8, 8-byte piece t), with the prefill kernel's
// conflict-free lane map.  Returns 0 or the code of the wait that ran out.
template <int A_STAGES, bool Q5, int RAW, int META>
__device__ __forceinline__ int tc_make_q4k(TcBarriers* bar, uint8_t* a_stage, uint8_t* a2_tile, const uint8_t* raw_stage, TcRowMeta* meta,
                                           int nb, int tiles_here, int wd, int lane)
{
    constexpr int kTcAStages = A_STAGES;
    int fail = 0;
    const int t = lane & 3, qd = lane >> 3, g = ((lane >> 2) & 1) ? (qd ^ 5) : qd;
    const bool unit_ok = wd < tiles_here;
    const uint32_t arow_off = (uint32_t)(2 * wd * 1024 + g * 128);
    const uint32_t col_lo = (uint32_t)((t ^ g) << 4), col_hi = (uint32_t)(((4 + t) ^ g) << 4);
    const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
    const __half2 km1024 = __half2half2(__ushort_as_half((unsigned short)0xE400)), km64 = __half2half2(__ushort_as_half((unsigned short)0xD400));
    for (int i = 0; i < nb && !fail; i++) {
        const int rs = i % RAW;
        if (!mbar_wait(&bar->raw_full[rs], ((uint32_t)i / RAW) & 1u)) { fail = 4; break; }
        // Q5: the Q5_K unit is the Q4_K unit plus a fifth-bit segment (lane 4g + t: qh[8t .. 8t+8) of rows g and g + 8); bit s
        // of qh[l] lifts value l of sub-block s by 16 (crates/ferric-gguf/src/lib.rs:690-716), the rest is Q4_K's arithmetic.
        constexpr int kUnitBytes = Q5 ? kQ5KUnit : kQ4KUnit;
        const uint8_t* u = raw_stage + rs * (8 * kUnitBytes) + wd * kUnitBytes;
        uint4 hdr[2], qs[2][2];
        uint2 q5[2];
#pragma unroll
        for (int hi = 0; hi < 2; hi++) {
            hdr[hi] = qs[hi][0] = qs[hi][1] = make_uint4(0, 0, 0, 0);
            q5[hi] = make_uint2(0, 0);
            if (unit_ok) {
                hdr[hi] = *reinterpret_cast<const uint4*>(u + 16 * (g + 8 * hi));
                qs[hi][0] = *reinterpret_cast<const uint4*>(u + 256 + 512 * (2 * hi) + 16 * (4 * g + t));
                qs[hi][1] = *reinterpret_cast<const uint4*>(u + 256 + 512 * (2 * hi + 1) + 16 * (4 * g + t));
                if (Q5) q5[hi] = *reinterpret_cast<const uint2*>(u + kQ5KOffQh + 16 * (4 * g + t) + 8 * hi);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar->raw_empty[rs]);
        // the rows' eight 6-bit scales and mins, one per byte (crates/ferric-gguf/src/lib.rs:795-804)
        uint32_t scb[2][2], mnb[2][2];
#pragma unroll
        for (int hi = 0; hi < 2; hi++) {
            scb[hi][0] = hdr[hi].y & 0x3F3F3F3Fu;
            scb[hi][1] = (hdr[hi].w & 0x0F0F0F0Fu) | ((hdr[hi].y >> 2) & 0x30303030u);
            mnb[hi][0] = hdr[hi].z & 0x3F3F3F3Fu;
            mnb[hi][1] = ((hdr[hi].w >> 4) & 0x0F0F0F0Fu) | ((hdr[hi].z >> 2) & 0x30303030u);
        }
        if (t < 2) {
            // the min step's A operand: A2[row][sb] = A2[row][8 + sb] = min of sub-block sb, in slot i & 3 (16-byte columns
            // 2 slot + t of the row).  That slot was last read by the min MMA of super-block i - 4, which completed before
            // any ring stage this warp has since been granted was released.
            uint8_t* arow = a2_tile + arow_off;
            const uint32_t col = (uint32_t)(((2 * (i & 3) + t) ^ g) << 4);
#pragma unroll
            for (int hi = 0; hi < 2; hi++) {
                uint4 mins;
                mins.x = tc_u32(__hsub2(tc_h2(__byte_perm(mnb[hi][0], 0x64u, 0x4140u)), k1024));   // mins 0, 1
                mins.y = tc_u32(__hsub2(tc_h2(__byte_perm(mnb[hi][0], 0x64u, 0x4342u)), k1024));   // mins 2, 3
                mins.z = tc_u32(__hsub2(tc_h2(__byte_perm(mnb[hi][1], 0x64u, 0x4140u)), k1024));
                mins.w = tc_u32(__hsub2(tc_h2(__byte_perm(mnb[hi][1], 0x64u, 0x4342u)), k1024));
                *reinterpret_cast<uint4*>(arow + hi * 1024 + col) = mins;
            }
        }
        if (t == 0) {   // hand (d, dmin) of this super-block's rows to the drain
#pragma unroll
            for (int hi = 0; hi < 2; hi++) {
                const float dv = __half2float(__ushort_as_half((unsigned short)(hdr[hi].x & 0xffffu)));
                const float dm = __half2float(__ushort_as_half((unsigned short)(hdr[hi].x >> 16)));
                *reinterpret_cast<float2*>(&meta[(i % META) * kTcRows + 16 * wd + 8 * hi + g]) = make_float2(dv, dm);
            }
        }
#pragma unroll
        for (int e = 0; e < 2 && !fail; e++) {       // a ring stage holds two K chunks
            const int c = 2 * i + e, s = c % kTcAStages;
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
                const int j = 2 * e + cc;
                uint4 lo[2], up8[2];
#pragma unroll
                for (int hi = 0; hi < 2; hi++) {
                    // sub-blocks 2j (low nibbles) and 2j + 1 (high nibbles): bytes 2j & 3, (2j + 1) & 3 of scale word j >> 1
                    const __half2 s0 = __hsub2(tc_bcast_byte(scb[hi][j >> 1], (2 * j) & 3), k1024);
                    const __half2 s1 = __hsub2(tc_bcast_byte(scb[hi][j >> 1], (2 * j + 1) & 3), k1024);
                    const uint4 q4 = qs[hi][j >> 1];
                    const uint32_t w0 = (j & 1) ? q4.z : q4.x, w1 = (j & 1) ? q4.w : q4.y;
                    if (Q5) {   // five-bit values, one per byte, then the byte form of the maker
                        const uint32_t l0 = (w0 & 0x0F0F0F0Fu) | (((q5[hi].x >> (2 * j)) & 0x01010101u) << 4);
                        const uint32_t l1 = (w1 & 0x0F0F0F0Fu) | (((q5[hi].y >> (2 * j)) & 0x01010101u) << 4);
                        const uint32_t u0 = ((w0 >> 4) & 0x0F0F0F0Fu) | (((q5[hi].x >> (2 * j + 1)) & 0x01010101u) << 4);
                        const uint32_t u1 = ((w1 >> 4) & 0x0F0F0F0Fu) | (((q5[hi].y >> (2 * j + 1)) & 0x01010101u) << 4);
                        lo[hi] = tc_make8_bytes(l0, l1, s0, __hmul2(s0, km1024));
                        up8[hi] = tc_make8_bytes(u0, u1, s1, __hmul2(s1, km1024));
                    } else {
                        tc_make16(w0, w1, s0, __hmul2(s0, km1024), s1, __hmul2(s1, km64), lo[hi], up8[hi]);
                    }
                }
                // (every lane polls: one polling lane plus a shuffle was measured 15 % slower -- the wake-up is on the critical path)
                if (cc == 0 && !mbar_wait(&bar->empty[s], (((uint32_t)c / kTcAStages) & 1u) ^ 1u)) { fail = 5; break; }
                uint8_t* arow = a_stage + (s * 2 + cc) * kTcABytes + arow_off;
#pragma unroll
                for (int hi = 0; hi < 2; hi++) {
                    *reinterpret_cast<uint4*>(arow + hi * 1024 + col_lo) = lo[hi];
                    *reinterpret_cast<uint4*>(arow + hi * 1024 + col_hi) = up8[hi];
                }
            }
            if (fail) break;
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->full[s]);   // also publishes this block's row meta and mins (written above)
        }
    }
    return fail;
}

// Four Q6_K weights (6-bit values in the bytes of q) times both scale digits -> f16 integers sl * (q - 32) and
// sh * (q - 32), in the order bytes 0, 2, 1, 3: (1024 + q) * s - 1056 s, exact as above (1056 s = 33 s * 32).
__device__ __forceinline__ void tc_make4_q6(uint32_t q, __half2 sl, __half2 bl, __half2 sh, __half2 bh, uint2& p0, uint2& p1)
{
    const __half2 a02 = tc_h2((q & 0x003F003Fu) | 0x64006400u), a13 = tc_h2(((q >> 8) & 0x003F003Fu) | 0x64006400u);
    p0 = make_uint2(tc_u32(__hfma2(a02, sl, bl)), tc_u32(__hfma2(a13, sl, bl)));
    p1 = make_uint2(tc_u32(__hfma2(a02, sh, bh)), tc_u32(__hfma2(a13, sh, bh)));
}

// Q6_K (unit layout in layout.h; lane ownership as in the prefill kernel's Q6_K stage): two operand planes per chunk,
// plane 0 = sl * (q - 32), plane 1 = sh * (q - 32) with sc = 16 sh + sl.  Row meta carries d only.
template <int A_STAGES, int CH, int RAW, int META>
__device__ __forceinline__ int tc_make_q6k(TcBarriers* bar, uint8_t* a_stage, const uint8_t* raw_stage, TcRowMeta* meta, int nb,
                                           int tiles_here, int wd, int lane)
{
    constexpr int kChunkBytes = 2 * kTcABytes;   // both planes of one K chunk
    int fail = 0;
    const int t = lane & 3, qd = lane >> 3, g = ((lane >> 2) & 1) ? (qd ^ 5) : qd;
    const bool unit_ok = wd < tiles_here;
    const uint32_t arow_off = (uint32_t)(2 * wd * 1024 + g * 128);
    const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400)), k1032 = __half2half2(__ushort_as_half((unsigned short)0x6408));
    const __half2 km1056 = __half2half2(__ushort_as_half((unsigned short)0xE420));
    for (int i = 0; i < nb && !fail; i++) {
        const int rs = i % RAW;
        if (!mbar_wait(&bar->raw_full[rs], ((uint32_t)i / RAW) & 1u)) { fail = 4; break; }
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
                const float dv = __half2float(__ushort_as_half((unsigned short)(hi ? (dpair >> 16) : (dpair & 0xffffu))));
                *reinterpret_cast<float2*>(&meta[(i % META) * kTcRows + 16 * wd + 8 * hi + g]) = make_float2(dv, 0.0f);
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
                const uint32_t slb = scw & 0x0F0F0F0Fu, shb = ((scw >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;   // digits sl, sh + 8
#pragma unroll
                for (int c = 0; c < 2; c++) {
#pragma unroll
                    for (int is = 0; is < 2; is++) {
                        const __half2 sl = __hsub2(tc_bcast_byte(slb, 2 * c + is), k1024);      // sc = 16 sh + sl, sl 0..15
                        const __half2 sh = __hsub2(tc_bcast_byte(shb, 2 * c + is), k1032);      // sh -8..7
                        const uint4 qlv = ql[hi][c];
                        const uint32_t lw = (2 * h + is) == 0 ? qlv.x : ((2 * h + is) == 1 ? qlv.y : ((2 * h + is) == 2 ? qlv.z : qlv.w));
                        const uint32_t hw = (2 * h + is) == 0 ? qh[hi].x : ((2 * h + is) == 1 ? qh[hi].y : ((2 * h + is) == 2 ? qh[hi].z : qh[hi].w));
                        const uint32_t q = ((lw >> (4 * kp)) & 0x0F0F0F0Fu) | (((hw >> (2 * (2 * kp + c))) & 0x03030303u) << 4);
                        tc_make4_q6(q, sl, __hmul2(sl, km1056), sh, __hmul2(sh, km1056), p0[hi][2 * c + is], p1[hi][2 * c + is]);
                    }
                }
            }
            // ring entry of this chunk: CH chunks share a stage; wait for it before its first chunk, hand it over after its last
            const int c4 = (4 * i + j) / CH, cc = j % CH, s = c4 % A_STAGES;
            if (cc == 0 && !mbar_wait(&bar->empty[s], (((uint32_t)c4 / A_STAGES) & 1u) ^ 1u)) { fail = 5; break; }
            uint8_t* arow = a_stage + (s * CH + cc) * kChunkBytes + arow_off;
#pragma unroll
            for (int hi = 0; hi < 2; hi++)
#pragma unroll
                for (int k = 0; k < 4; k++) {   // k = 2c + is: 16-byte column 2k + (t >> 1), half t & 1
                    const uint32_t off = (uint32_t)(hi * 1024 + (((2 * k + (t >> 1)) ^ g) << 4) + 8 * (t & 1));
                    *reinterpret_cast<uint2*>(arow + off) = p0[hi][k];
                    *reinterpret_cast<uint2*>(arow + kTcABytes + off) = p1[hi][k];
                }
            if (cc == CH - 1) {
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar->full[s]);
            }
        }
    }
    return fail;
}

template <uint32_t TY, int N_TILE>
__global__ void __launch_bounds__(kTcThreads, 1)
gemv_tc_kernel(const uint8_t* __restrict__ units, const __grid_constant__ CUtensorMap xmap, const __half* __restrict__ sbsum,
               const float* __restrict__ up, float* __restrict__ out, size_t ld_out, size_t split_stride, int rows, int nblk,
               int m, int m_pad, int row_tiles16, int blocks_per_split, int gu16, int* __restrict__ err)
{
    // gu16 > 0: the matrix is [gate rows | up rows] of gu16 sixteen-row units each, this CTA takes 64 gate rows and the
    // 64 up rows of the same outputs, and the drain stores silu(gate) * up (rows / 2 a multiple of 64, no K split).
    extern __shared__ uint8_t tc_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int kStages = tc_stages(TY, N_TILE), kBBytes = tc_b_bytes(N_TILE), kActs = N_TILE / kTcLimbs;
    // accumulator sets in tensor memory (each two accumulators wide): as many as its 512 columns hold, so that at the
    // narrow tile the MMAs run up to four super-blocks ahead of the drain
    constexpr int kAcc = 256 / N_TILE;
    constexpr int kCh = tc_chunks(TY, N_TILE), kPlanes = tc_planes(TY), kAStageBytes = kCh * kPlanes * kTcABytes, kBStageBytes = kCh * kBBytes;
    constexpr int kUnit = tc_unit_bytes(TY), kTcRawBytes = tc_raw_bytes(TY);
    uint8_t* a_stage = smem;                                  // [kStages][kCh][kPlanes][16384]
    uint8_t* b_stage = a_stage + kStages * kAStageBytes;      // [kStages][kCh][N_TILE * 128]
    uint8_t* a2_tile = b_stage + kStages * kBStageBytes;      // Q4_K, Q5_K: the min step's operands
    uint8_t* b2_tile = a2_tile + (tc_has_mins(TY) ? kTcABytes : 0);
    uint8_t* raw_stage = a2_tile + tc_min_bytes(TY, N_TILE);
    constexpr int kRaw = tc_raw_stages(TY, N_TILE), kMeta = tc_meta_stages(N_TILE);
    TcRowMeta* meta = reinterpret_cast<TcRowMeta*>(raw_stage + kRaw * kTcRawBytes);   // [kMeta][128]
    float* sums = reinterpret_cast<float*>(meta + kMeta * kTcRows);   // [2][kActs]: staged UP of a super-block
    TcBarriers* bar = reinterpret_cast<TcBarriers*>(sums + 2 * kTcSumFloats);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kTcRows, rt0 = blockIdx.x * 8, act0 = blockIdx.y * kActs;
    const int tiles_here = gu16 > 0 ? 8 : max(0, min(8, row_tiles16 - rt0));
    const int blk0 = blockIdx.z * blocks_per_split, nb = max(0, min(nblk, blk0 + blocks_per_split) - blk0);

    if (threadIdx.x == 0) {
        for (int i = 0; i < kRaw; i++) {
            mbar_init(&bar->raw_full[i], 1);
            mbar_init(&bar->raw_empty[i], kTcMakerWarps);
        }
        for (int i = 0; i < kStages; i++) {
            mbar_init(&bar->full[i], kTcMakerWarps + 1);
            mbar_init(&bar->empty[i], 1);
        }
        for (int i = 0; i < kAcc; i++) {
            mbar_init(&bar->acc_full[i], 1);
            mbar_init(&bar->acc_empty[i], kTcDrainWarps);
        }
        bar->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // kAcc sets of two accumulators (Q4_K: product and min term; Q6_K: one per operand plane); a power of two >= 128
    constexpr int kTmemCols = kAcc * 2 * N_TILE;
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
                const int rs = i % kRaw;
                if (!mbar_wait(&bar->raw_empty[rs], (((uint32_t)i / kRaw) & 1u) ^ 1u)) { fail = 1; break; }
                mbar_expect_tx(&bar->raw_full[rs], (uint32_t)(tiles_here * kUnit));
                for (int t = 0; t < tiles_here; t++) {
                    const int rt = gu16 > 0 ? (t < 4 ? 4 * (int)blockIdx.x + t : gu16 + 4 * (int)blockIdx.x + t - 4) : rt0 + t;
                    bulk_g2s(raw_stage + rs * kTcRawBytes + t * kUnit, units + ((size_t)rt * nblk + blk0 + i) * kUnit, kUnit,
                             &bar->raw_full[rs]);
                }
            }
        }
    } else if (warp == 2) {
        // ---------------- limb producer: [64 k x N_TILE operand rows] f16 per stage
        if (lane == 0) {
            pdl_wait();   // the limbs come from the preparation kernel launched just before
            uint32_t s = 0, ph = 0;
            for (int c = 0; c < (4 / kCh) * nb; c++) {
                if (!mbar_wait(&bar->empty[s], ph ^ 1u)) { fail = 2; break; }
                mbar_expect_tx(&bar->full[s], (uint32_t)kBStageBytes);
#pragma unroll
                for (int cc = 0; cc < kCh; cc++)
                    tma_load_2d(b_stage + s * kBStageBytes + cc * kBBytes, &xmap, (4 * blk0 + kCh * c + cc) * kTcChunkK, kTcLimbs * act0,
                                &bar->full[s]);
                if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: four K chunks per super-block into accumulator set (i & 1).  This one thread's
        // instruction stream paces the kernel at narrow tiles, so it is kept lean: running stage counters instead of
        // modulo / division, barrier addresses and descriptor low words advanced by adds.
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(kTcRows, N_TILE);
            const uint32_t full0 = smem_u32(&bar->full[0]), empty0 = smem_u32(&bar->empty[0]);
            const uint32_t adesc0 = umma_desc_lo(smem_u32(a_stage)), bdesc0 = umma_desc_lo(smem_u32(b_stage));
            uint32_t sa = 0, pa = 0;     // stage and phase parity of the ring
            const uint32_t a2desc = umma_desc_lo(smem_u32(a2_tile)), b2desc = umma_desc_lo(smem_u32(b2_tile));
            for (int i = 0; i < nb && !fail; i++) {
                const int buf = i % kAcc;
                // (the drain arrives once on every set before its loop, after it has staged the first super-blocks'
                // sub-block sums: every wait here is a real one)
                if (!mbar_wait(&bar->acc_empty[buf], ((uint32_t)i / kAcc) & 1u)) { fail = 3; break; }
                tc_fence_after();
                const uint32_t d0 = tmem_acc + (uint32_t)(buf * 2 * N_TILE);
#pragma unroll
                for (int e = 0; e < 4 / kCh; e++) {
                    if (!mbar_try(full0 + 8 * sa, pa) && !mbar_wait(&bar->full[sa], pa)) { fail = 3; break; }
                    tc_fence_after();
#pragma unroll
                    for (int cc = 0; cc < kCh; cc++) {
                        const uint32_t ad = adesc0 + (sa * (uint32_t)kCh + cc) * (uint32_t)((kPlanes * kTcABytes) >> 4);
                        const uint32_t bd = bdesc0 + (sa * (uint32_t)kCh + cc) * (uint32_t)(kBBytes >> 4);
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++)
#pragma unroll
                            for (int pl = 0; pl < kPlanes; pl++)
                                umma_f16_lo(d0 + pl * N_TILE, ad + (uint32_t)(pl * (kTcABytes >> 4) + 2 * k4), bd + 2 * k4, idesc,
                                            (e | cc | k4) ? 1u : 0u);
                    }
                    if (tc_has_mins(TY) && e == 4 / kCh - 1)   // mins x sub-block sums, K = 16 (operands in place since the first chunk / since acc_empty)
                        umma_f16_lo(d0 + N_TILE, a2desc + 2 * (uint32_t)(i & 3), b2desc + 2 * (uint32_t)(i % kAcc), idesc, 0u);
                    umma_commit_addr(empty0 + 8 * sa);
                    if (++sa == (uint32_t)kStages) { sa = 0; pa ^= 1u; }
                }
                if (!fail) umma_commit(&bar->acc_full[buf]);
            }
        }
    } else if (warp < kTcFirstDrain) {
        // ---------------- operand makers (per quant type, above)
        const int wd = warp - kTcFirstMaker;
        if (TY == kGgmlQ4K) fail = tc_make_q4k<kStages, false, kRaw, kMeta>(bar, a_stage, a2_tile, raw_stage, meta, nb, tiles_here, wd, lane);
        else if (TY == kGgmlQ5K) fail = tc_make_q4k<kStages, true, kRaw, kMeta>(bar, a_stage, a2_tile, raw_stage, meta, nb, tiles_here, wd, lane);
        else fail = tc_make_q6k<kStages, kCh, kRaw, kMeta>(bar, a_stage, raw_stage, meta, nb, tiles_here, wd, lane);
    } else {
        // ---------------- drain: TMEM lane = weight row; columns 2b, 2b + 1 = the hi and lo limb of activation row act0 + b.
        // Two warps share a TMEM lane quarter; warp half h takes the groups of eight activation rows 2g + h.
        const int q = warp & 3, rloc = 32 * q + lane, wrow = row0 + rloc, half = (warp - kTcFirstDrain) >> 2;
        constexpr int kGroups = N_TILE / 32;           // groups of eight activation rows (16 columns) per drain warp
        float acc[kGroups * 8];
#pragma unroll
        for (int b = 0; b < kGroups * 8; b++) acc[b] = 0.0f;
        pdl_wait();   // up comes from the preparation kernel
        // The activation rows' scales of a super-block are fetched one super-block ahead into a register and staged in
        // shared memory.
        const int dt = threadIdx.x - 32 * kTcFirstDrain;          // 0..255
        auto fetch = [&](int i) {
            float uv = 0.f;
            if (i < nb && dt < kActs) uv = __ldg(up + (size_t)(blk0 + i) * m_pad + act0 + dt);
            return uv;
        };
        // The min step's B operand: 16 f16 per operand row and super-block (two 16-byte pieces), copied by the drain
        // threads into slot i mod kAcc of the B2 tile kAcc super-blocks ahead -- the slot's last reader, the min MMA of
        // super-block i, has completed when acc_full(i) fires, and the copy is published by this iteration's acc_empty
        // arrival, which the MMAs of super-block i + kAcc wait for.
        auto load_b2 = [&](int i) {
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (tc_has_mins(TY) && i < nb && dt < 2 * N_TILE && kTcLimbs * act0 + (dt >> 1) < kTcLimbs * m)
                val = __ldg(reinterpret_cast<const uint4*>(sbsum + ((size_t)(blk0 + i) * m_pad * kTcLimbs + kTcLimbs * act0 + (dt >> 1)) * 16) +
                            (dt & 1));
            return val;
        };
        auto store_b2 = [&](int i, const uint4& val) {
            if (!tc_has_mins(TY) || i >= nb || dt >= 2 * N_TILE) return;
            const int r = dt >> 1, c = dt & 1;
            *reinterpret_cast<uint4*>(b2_tile + r * 128 + (((2 * (i % kAcc) + c) ^ (r & 7)) << 4)) = val;
        };
        float uv = fetch(0);
        if (dt < kActs) sums[dt] = uv;
#pragma unroll
        for (int i = 0; i < kAcc; i++) store_b2(i, load_b2(i));
        fence_proxy_async();
        named_bar_sync(1, 32 * kTcDrainWarps);
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < kAcc; i++) mbar_arrive(&bar->acc_empty[i]);
        }
        const uint32_t lane_base = tmem_acc + ((uint32_t)(32 * q) << 16);
        for (int i = 0; i < nb && !fail; i++) {
            const int buf = i % kAcc;
            uv = fetch(i + 1);
            const uint4 b2v = load_b2(i + kAcc);   // in flight under the wait and the accumulator reads below
            if (!mbar_wait(&bar->acc_full[buf], ((uint32_t)i / kAcc) & 1u)) { fail = 6; break; }
            tc_fence_after();
            const TcRowMeta rm = meta[(i % kMeta) * kTcRows + rloc];
            const float* sl = sums + (i & 1) * kTcSumFloats;
            const float ndmin = -rm.dmin;
#pragma unroll
            for (int gg = 0; gg < kGroups; gg++) {
                const int grp = 2 * gg + half;
                uint32_t v[16], w[16];
                const uint32_t c0 = lane_base + (uint32_t)(buf * 2 * N_TILE + 16 * grp);
                tmem_ld_16x2(c0, c0 + (uint32_t)N_TILE, v, w);
#pragma unroll
                for (int bb = 0; bb < 8; bb++) {
                    const float scale = sl[8 * grp + bb];
                    if (tc_has_mins(TY)) {     // w = the min term's accumulator
                        const float V = fmaf(__uint_as_float(v[2 * bb + 1]), 0.00048828125f, __uint_as_float(v[2 * bb]));
                        const float Mn = fmaf(__uint_as_float(w[2 * bb + 1]), 0.00048828125f, __uint_as_float(w[2 * bb]));
                        acc[8 * gg + bb] = fmaf(scale, fmaf(rm.d, V, ndmin * Mn), acc[8 * gg + bb]);
                    } else {                   // w = the second scale digit's plane: D1 + 16 D2
                        const float hi = fmaf(16.0f, __uint_as_float(w[2 * bb]), __uint_as_float(v[2 * bb]));
                        const float lo = fmaf(16.0f, __uint_as_float(w[2 * bb + 1]), __uint_as_float(v[2 * bb + 1]));
                        acc[8 * gg + bb] = fmaf(scale * rm.d, fmaf(lo, 0.00048828125f, hi), acc[8 * gg + bb]);
                    }
                }
            }
            // every drain thread has finished reading the other slot (it did so one iteration ago and has met the
            // barrier below since), so the next super-block's values can go there
            if (dt < kActs) sums[((i + 1) & 1) * kTcSumFloats + dt] = uv;
            store_b2(i + kAcc, b2v);
            fence_proxy_async();
            named_bar_sync(1, 32 * kTcDrainWarps);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->acc_empty[buf]);
        }
        if (gu16 > 0) {
            // TMEM lanes 0..63 hold gate rows, 64..127 the up rows of the same outputs: the up half hands its sums over
            // through shared memory (the operand ring is idle by now: every MMA has completed)
            float* xch = reinterpret_cast<float*>(a_stage);       // [kActs][64]
            if (q >= 2 && !fail) {
#pragma unroll
                for (int gg = 0; gg < kGroups; gg++)
#pragma unroll
                    for (int bb = 0; bb < 8; bb++) xch[(8 * (2 * gg + half) + bb) * 64 + rloc - 64] = acc[8 * gg + bb];
            }
            named_bar_sync(1, 32 * kTcDrainWarps);
            if (q < 2 && !fail) {
                const size_t col = (size_t)blockIdx.x * 64 + rloc;
#pragma unroll
                for (int gg = 0; gg < kGroups; gg++)
#pragma unroll
                    for (int bb = 0; bb < 8; bb++) {
                        const int al = 8 * (2 * gg + half) + bb, act = act0 + al;
                        if (act < m) out[(size_t)act * ld_out + col] = silu_mul(acc[8 * gg + bb], xch[al * 64 + rloc]);
                    }
            }
        } else if (!fail && wrow < rows) {
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

// The same sum of the K pieces, stored not into y but -- as step 1 of the two-step pushed all-reduce (kernels_tpwide.cu) --
// into the stage-1 region of the rank that owns each slice of the flat [m x rows] result: the product scatters itself.
__global__ void tc_finish_scatter_kernel(const float* __restrict__ part, int splits, size_t split_stride, size_t n, WideDst dst)
{
    pdl_launch_dependents();
    pdl_wait();
    const unsigned stamp = wide_stamp(dst.epoch);
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
        float4 v = *reinterpret_cast<const float4*>(part + i);
        for (int s = 1; s < splits; s++) {
            const float4 t = *reinterpret_cast<const float4*>(part + s * split_stride + i);
            v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
        }
        const size_t owner = i / dst.slice, off = i - owner * dst.slice;
        uint2* base = nullptr;
#pragma unroll
        for (int r = 0; r < kMaxRanks; r++)
            if ((size_t)r == owner) base = dst.stage1[r];   // static indices keep the table in the parameter space
        store_pairs4(base + (size_t)(stamp & 1) * dst.parity_stride1 + off, v, stamp);
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
    size_t off_sb, off_up, off_part, total;   // scratch offsets (XL at 0)
    bool needs_finish, fused_swiglu;
};

TcPlan tc_plan(uint32_t ty, const DeviceWeights& w, size_t m, Epilogue epi, int sm_count)
{
    TcPlan p;
    p.n_tile = m <= 32 ? 64 : 128;   // operand rows per tile: 32 or 64 activation rows (tensor memory holds 4 x n_tile columns)
    const size_t row_tiles = (w.rows + kTcRows - 1) / kTcRows, act_tiles = (kTcLimbs * m + p.n_tile - 1) / p.n_tile;
    const size_t tiles = row_tiles * act_tiles;
    // Cut K so that the CTAs come in whole waves: the cost of a cut is the number of waves times the super-blocks of one
    // CTA (plus two for filling and emptying its pipeline).
    size_t splits = 1, best = ~(size_t)0;
    for (size_t s = 1; s <= 16 && s <= w.nblk; s++) {
        const size_t waves = (tiles * s + (size_t)sm_count - 1) / (size_t)sm_count;
        const size_t cost = 2 * waves * ((w.nblk + s - 1) / s + 2) + s;   // each piece also costs the finish kernel half a super-block
        if (cost < best) {
            best = cost;
            splits = s;
        }
    }
    p.blocks_per_split = (int)((w.nblk + splits - 1) / splits);
    p.splits = (int)((w.nblk + p.blocks_per_split - 1) / p.blocks_per_split);
    p.fused_swiglu = epi == kEpiSwiglu && p.splits == 1 && w.rows % 128 == 0;   // the kernel's own gate / up pairing
    p.needs_finish = p.splits > 1 || (epi == kEpiSwiglu && !p.fused_swiglu);
    p.m_pad = act_tiles * (size_t)(p.n_tile / kTcLimbs);
    p.off_sb = align256(kTcLimbs * m * w.cols * sizeof(__half));
    p.off_up = p.off_sb + (tc_has_mins(ty) ? align256(kTcLimbs * p.m_pad * w.nblk * 16 * sizeof(__half)) : 0);
    p.off_part = p.off_up + align256(p.m_pad * w.nblk * sizeof(float));
    p.total = p.off_part + (p.needs_finish ? align256((size_t)p.splits * m * w.rows * sizeof(float)) : 0);
    return p;
}

template <uint32_t TY, int N_TILE>
int32_t launch_tc_tile(cudaStream_t st, const DeviceWeights& w, const CUtensorMap& map, const __half* sb, const float* up,
                       float* out, size_t ld_out, size_t split_stride, size_t m, const TcPlan& p, bool pdl)
{
    static bool attr_done[64] = {};
    int dev = 0;
    FERRIC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !attr_done[dev]) {
        FERRIC_CUDA_TRY(cudaFuncSetAttribute(gemv_tc_kernel<TY, N_TILE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             tc_smem_bytes(TY, N_TILE)));
        attr_done[dev] = true;
    }
    dim3 grid((unsigned)((w.rows + kTcRows - 1) / kTcRows), (unsigned)((kTcLimbs * m + N_TILE - 1) / N_TILE), (unsigned)p.splits);
    FERRIC_CUDA_TRY(launch_kernel(gemv_tc_kernel<TY, N_TILE>, grid, dim3(kTcThreads), (size_t)tc_smem_bytes(TY, N_TILE), st, pdl,
                                  (const uint8_t*)w.units, map, sb, up, out, ld_out, split_stride, (int)w.rows, (int)w.nblk,
                                  (int)m, (int)p.m_pad, (int)w.row_tiles(), p.blocks_per_split,
                                  p.fused_swiglu ? (int)(w.rows / 32) : 0, gemm_status_word()));
    return kOk;
}
}  // namespace

bool gemv_tc_eligible(uint32_t ty, const DeviceWeights& w, size_t m)
{
    // Measured cross-over with the mma.sync GEMV, which runs in passes of 4 activation rows (us per product, GEMV / this
    // kernel: gate|up 34816 x 5120 at 8 rows 50 / 63, at 9 rows 71 / 63; q|k|v at 9 rows 24 / 22; down Q6_K 5120 x 17408
    // at 12 rows 59 / 64, at 13 rows 71 / 64): Q4_K (and Q5_K, the same kernel) from 9 rows, Q6_K from 13.
    // FERRIC_CUDA_GEMV_TC_MIN_M overrides both; 0 disables the path.
    const char* env = getenv("FERRIC_CUDA_GEMV_TC_MIN_M");   // read per call: tests move the threshold
    const int forced = env ? atoi(env) : -1;
    if (ty != kGgmlQ4K && ty != kGgmlQ5K && ty != kGgmlQ6K) return false;
    const int min_m = forced >= 0 ? forced : (ty == kGgmlQ6K ? 13 : 9);
    return min_m > 0 && m >= (size_t)min_m && m <= 4096 && w.nblk > 0 && w.rows > 0 && w.rows <= (size_t)INT32_MAX / 2;
}

size_t gemv_tc_scratch_bytes(uint32_t ty, const DeviceWeights& w, size_t m, Epilogue epi, int sm_count)
{
    return tc_plan(ty, w, m, epi, sm_count).total;
}

int32_t launch_gemv_tc(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const float* x, size_t m, size_t ldx, float* y, size_t ldy,
                       Epilogue epi, void* scratch, const GemvTuning& tune, int* launches, const WideDst* scatter, bool* scattered)
{
    if (scattered) *scattered = false;
    EncodeTiledFn enc = tc_encode_fn();
    if (!enc) {
        set_last_error("the CUDA driver does not export cuTensorMapEncodeTiled");
        return kErrCuda;
    }
    const TcPlan p = tc_plan(ty, w, m, epi, tune.sm_count);
    uint8_t* base = reinterpret_cast<uint8_t*>(scratch);
    __half* xl = reinterpret_cast<__half*>(base);
    __half* sb = tc_has_mins(ty) ? reinterpret_cast<__half*>(base + p.off_sb) : nullptr;
    float* up = reinterpret_cast<float*>(base + p.off_up);
    float* part = reinterpret_cast<float*>(base + p.off_part);

    const size_t pairs = (m + 1) / 2, warps = pairs * w.nblk;
    FERRIC_CUDA_TRY(launch_kernel(tc_prep_kernel, dim3((unsigned)((warps + kTcPrepWarps - 1) / kTcPrepWarps)), dim3(32 * kTcPrepWarps),
                                  0, st, tune.pdl, x, m, p.m_pad, ldx, w.nblk, xl, w.cols, sb, up));
    CUtensorMap map;
    const cuuint32_t box[2] = {(cuuint32_t)kTcChunkK, (cuuint32_t)p.n_tile};
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t dims[2] = {(cuuint64_t)w.cols, (cuuint64_t)(kTcLimbs * m)};
        const cuuint64_t strides[1] = {(cuuint64_t)w.cols * 2};
        CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xl, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            set_last_error("cuTensorMapEncodeTiled (limbs) failed with code %d", (int)r);
            return kErrCuda;
        }
    }
    float* out = p.needs_finish ? part : y;
    const size_t ld_out = p.needs_finish ? w.rows : ldy, split_stride = m * w.rows;
    int32_t rc;
    if (ty == kGgmlQ6K) {
        if (p.n_tile == 64) rc = launch_tc_tile<kGgmlQ6K, 64>(st, w, map, sb, up, out, ld_out, split_stride, m, p, tune.pdl);
        else rc = launch_tc_tile<kGgmlQ6K, 128>(st, w, map, sb, up, out, ld_out, split_stride, m, p, tune.pdl);
    } else if (ty == kGgmlQ5K) {
        if (p.n_tile == 64) rc = launch_tc_tile<kGgmlQ5K, 64>(st, w, map, sb, up, out, ld_out, split_stride, m, p, tune.pdl);
        else rc = launch_tc_tile<kGgmlQ5K, 128>(st, w, map, sb, up, out, ld_out, split_stride, m, p, tune.pdl);
    } else {
        if (p.n_tile == 64) rc = launch_tc_tile<kGgmlQ4K, 64>(st, w, map, sb, up, out, ld_out, split_stride, m, p, tune.pdl);
        else rc = launch_tc_tile<kGgmlQ4K, 128>(st, w, map, sb, up, out, ld_out, split_stride, m, p, tune.pdl);
    }
    if (rc != kOk) return rc;
    *launches += 2;
    if (p.needs_finish && scatter && epi == kEpiStore && w.rows % 4 == 0) {
        // the K pieces are summed straight into the slice owners' memory (the flat result has row stride w.rows)
        const size_t n = m * w.rows;
        unsigned blocks = (unsigned)((n / 4 + 255) / 256);
        if (blocks > 4u * (unsigned)tune.sm_count) blocks = 4u * (unsigned)tune.sm_count;
        FERRIC_CUDA_TRY(launch_kernel(tc_finish_scatter_kernel, dim3(blocks), dim3(256), 0, st, tune.pdl, (const float*)part, p.splits,
                                      split_stride, n, *scatter));
        *launches += 1;
        if (scattered) *scattered = true;
    } else if (p.needs_finish) {
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
