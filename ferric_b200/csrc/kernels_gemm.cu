// Prefill (M >= 128) Q4_K x bf16 GEMM on the 5th-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory.
//
// Replaces Tensor::matmul_q4_k_coop (crates/ferric-tensor/src/dtype.rs:1818-1834, kernel :2059-2096):
// there a workgroup dequantises an 8x8 weight tile into shared memory and feeds 8x8x8 f32
// cooperative-matrix ops (Metal only; "exactly 1.0x" on NVIDIA, crates/ferric-core/src/lib.rs:90-100).
// Here a CTA owns 128 weight rows x 128, 256 or 512 activation rows (512 = all of tensor memory); above 256
// activation rows two CTAs on neighbouring SMs form a pair (cta_group::2) that works on a 256 x 512 tile: each
// dequantises its own 128 weight rows, each loads half of the activation tile, one thread of the leader issues
// M = 256 MMAs that read both CTAs' shared memory and write both CTAs' tensor memory.  That halves the
// activation bytes a CTA pulls from L2 per flop, which is what bounds the single-CTA form.
//   * warp 0 (one lane)  weight producer: bulk-copies the raw quant units of the next super-blocks;
//   * warp 2 (one lane)  activation producer: TMA-loads the activation tile (bf16 [rows, 64] boxes, 128-byte
//                        swizzle) of each 64-wide K chunk, as many chunks ahead as shared memory holds;
//   * warps 3..10        dequantise: each warp owns one 16-row unit, each thread 32 weights per K chunk, into
//                        bf16 with the reference decoder's exact arithmetic (d*sc, dmin*m, d1*q - mm, round to
//                        nearest even), stored into the K-major, 128-byte-swizzled A tile;
//   * warp 1 (one lane)  issues tcgen05.mma (N <= 256, K 16, bf16 -> f32 in TMEM), four or eight per chunk, and
//                        commits to the mbarriers that free the A / B stages (in both CTAs of a pair);
//   * warps 3..10        epilogue: tcgen05.ld the accumulator (lane = weight row, column = activation row),
//                        stage it in shared memory and TMA-store y[activation row][weight row].
// Every wait on an mbarrier is bounded: on expiry the thread records an error code and the CTA drains.
// No load in this file uses cluster multicast; the only multicast is tcgen05.commit's arrival on both CTAs'
// barriers.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"
#include "layout.h"
#include "tc_common.cuh"

namespace ferric {

constexpr int kGemmRows = 128;        // weight rows per CTA (UMMA M)
constexpr int kGemmChunkK = 64;       // K per pipeline stage: 64 bf16 = one 128-byte swizzle row
constexpr int kGemmStages = 3;        // dequantised A stages in flight
constexpr int kGemmRawStages = 2;     // raw quant super-blocks in flight
constexpr int kGemmDeqWarps = 8;      // one per 16-row unit of the 128-row tile
constexpr int kGemmHalves = 2;        // the two 8-row halves of its unit a dequant warp converts
constexpr int kGemmFirstDeqWarp = 3;                   // warp 0 weight producer, 1 MMA issuer, 2 activation producer
constexpr int kGemmThreads = 32 * (kGemmFirstDeqWarp + kGemmDeqWarps);
// raw quant bytes of one stage: 8 row tiles x one super-block (18432 for Q4_K, 22528 for Q5_K, 26880 for Q6_K)
__host__ __device__ constexpr int gemm_unit_bytes(uint32_t ty) { return ty == kGgmlQ4K ? kQ4KUnit : ty == kGgmlQ5K ? kQ5KUnit : kQ6KUnit; }
// Q8_0 is stored as planes ([rows][cols] int8 and [rows][cols/32] f16); a stage holds the tile of 128 rows x 256 columns
// of the first (32 KB, fetched as one TMA box) and its 128 x 8 scales (2 KB, a second box).
constexpr int kGemmQ8QsBytes = kGemmRows * 256, kGemmQ8DBytes = kGemmRows * 16;
__host__ __device__ constexpr int gemm_raw_bytes(uint32_t ty)
{
    return ty == kGgmlQ8_0 ? kGemmQ8QsBytes + kGemmQ8DBytes : 8 * gemm_unit_bytes(ty);
}
constexpr int kGemmABytes = kGemmRows * 128;                  // 16384 per stage
constexpr int kGemmStoreBytes = 32 * kGemmRows * 4;            // one [32 activation rows][128 weight rows] f32 store tile

// Activation bytes of one K chunk held by one CTA: the whole [n_tile x 64] bf16 tile, or half of it when two
// CTAs form a pair and each supplies half of the tensor core's B operand.
__host__ __device__ constexpr int gemm_b_bytes(int n_tile, bool pair = false) { return n_tile * 128 / (pair ? 2 : 1); }
// Activation stages: as many as the shared memory left by the A ring and the raw ring holds, at most 8.  What
// bounds the kernel at small N is bytes in flight (a stage's round trip through TMA and L2 is over a microsecond),
// so the ring is as deep as it can be: 8 stages at N 128, 4 at 256, 2 at 512.
constexpr int kGemmSmemMax = 232448;  // 227 KB per CTA
constexpr int kGemmMaxBStages = 8;
__host__ __device__ constexpr int gemm_fixed_bytes(uint32_t ty)
{
    return 1024 /*align*/ + 256 /*barriers*/ + kGemmStages * kGemmABytes + kGemmRawStages * gemm_raw_bytes(ty);
}
__host__ __device__ constexpr int gemm_b_stages(uint32_t ty, int n_tile, bool pair)
{
    return (kGemmSmemMax - gemm_fixed_bytes(ty)) / gemm_b_bytes(n_tile, pair) > kGemmMaxBStages
               ? kGemmMaxBStages
               : (kGemmSmemMax - gemm_fixed_bytes(ty)) / gemm_b_bytes(n_tile, pair);
}
// The narrow tile (at most 128 activation rows, where a K chunk's four MMAs are short and the MMA thread's barrier
// waits and commits -- about a hundred cycles each -- pace the kernel) runs ONE ring for both operands with two K chunks
// per stage: a stage is filled under one barrier (the dequant warps' arrivals + the activation producer's expect-tx)
// and released by one tcgen05.commit, a quarter of the hand-overs of the two-ring form.
// The paired 512-wide tile runs one ring too (one chunk per stage, three stages): its eight MMAs per chunk keep the tensor
// pipe busy for about as long as the issuing thread needs for them plus four waits / commits, so halving those leaves slack.
__host__ __device__ constexpr bool gemm_merged(int n_tile, bool pair)
{
    return (n_tile == 128 && !pair) || (n_tile == 256 && !pair) || (n_tile == 512 && pair);
}
__host__ __device__ constexpr int gemm_merged_chunks(int n_tile) { return n_tile == 128 ? 2 : 1; }
__host__ __device__ constexpr int gemm_merged_stages(int n_tile) { return n_tile == 128 ? 2 : 3; }
__host__ __device__ constexpr int gemm_smem_bytes(uint32_t ty, int n_tile, bool pair)
{
    return gemm_merged(n_tile, pair)
               ? 1024 + 256 + kGemmRawStages * gemm_raw_bytes(ty) +
                     gemm_merged_stages(n_tile) * gemm_merged_chunks(n_tile) * (kGemmABytes + gemm_b_bytes(n_tile, pair))
               : gemm_fixed_bytes(ty) + gemm_b_stages(ty, n_tile, pair) * gemm_b_bytes(n_tile, pair);
}
static_assert(gemm_smem_bytes(kGgmlQ4K, 256, false) <= kGemmSmemMax && gemm_smem_bytes(kGgmlQ6K, 256, false) <= kGemmSmemMax &&
                  gemm_smem_bytes(kGgmlQ8_0, 256, false) <= kGemmSmemMax && gemm_smem_bytes(kGgmlQ4K, 512, true) <= kGemmSmemMax && gemm_smem_bytes(kGgmlQ5K, 512, true) <= kGemmSmemMax &&
                  gemm_smem_bytes(kGgmlQ6K, 512, true) <= kGemmSmemMax && gemm_smem_bytes(kGgmlQ8_0, 512, true) <= kGemmSmemMax,
              "the merged ring of the paired tile fits");
static_assert(gemm_smem_bytes(kGgmlQ4K, 128, false) <= kGemmSmemMax && gemm_smem_bytes(kGgmlQ5K, 128, false) <= kGemmSmemMax &&
                  gemm_smem_bytes(kGgmlQ6K, 128, false) <= kGemmSmemMax && gemm_smem_bytes(kGgmlQ8_0, 128, false) <= kGemmSmemMax,
              "the merged ring fits");
static_assert(gemm_merged_stages(128) <= kGemmStages && gemm_merged_stages(512) <= kGemmStages, "barrier slots");
static_assert(gemm_merged_stages(128) * gemm_merged_chunks(128) * gemm_b_bytes(128) >= 4 * 32 * 128 * 4 &&
                  gemm_merged_stages(256) * gemm_b_bytes(256) >= 4 * 32 * 128 * 4 &&
                  gemm_merged_stages(512) * gemm_b_bytes(512, true) >= 4 * 32 * 128 * 4,
              "store staging fits the merged rings");
static_assert(gemm_b_stages(kGgmlQ4K, 128, false) == 8 && gemm_b_stages(kGgmlQ4K, 256, false) == 4 &&
                  gemm_b_stages(kGgmlQ4K, 512, false) == 2 && gemm_b_stages(kGgmlQ4K, 512, true) == 4,
              "Q4_K stage counts");
static_assert(gemm_b_stages(kGgmlQ5K, 128, false) >= 7 && gemm_b_stages(kGgmlQ5K, 256, false) >= 3 &&
                  gemm_b_stages(kGgmlQ5K, 512, false) >= 1 && gemm_b_stages(kGgmlQ5K, 512, true) >= 3,
              "Q5_K stage counts");
static_assert(gemm_b_stages(kGgmlQ6K, 128, false) == 7 && gemm_b_stages(kGgmlQ6K, 256, false) == 3 &&
                  gemm_b_stages(kGgmlQ6K, 512, true) == 3,
              "Q6_K stage counts");
// The epilogue stages its stores in the activation ring: two groups x two [32][128] f32 tiles.
static_assert(gemm_b_stages(kGgmlQ8_0, 128, false) >= 3 && gemm_b_stages(kGgmlQ8_0, 256, false) >= 3 &&
                  gemm_b_stages(kGgmlQ8_0, 512, true) >= 3,
              "Q8_0 stage counts (its 512-wide tile exists only in the paired form)");
static_assert(gemm_b_stages(kGgmlQ8_0, 256, false) * gemm_b_bytes(256) >= 4 * 32 * 128 * 4, "store staging fits");

// ---------------------------------------------------------------- the kernel
struct GemmBarriers {
    uint64_t raw_full[kGemmRawStages], raw_empty[kGemmRawStages];
    uint64_t a_full[kGemmStages], a_empty[kGemmStages], b_full[kGemmMaxBStages], b_empty[kGemmMaxBStages];
    uint64_t acc_full;
    uint32_t tmem_base;
    int abort;
};

// Exact float of an integer below 2^23 without the conversion unit: 0x4B000000 | v is 2^23 + v.
__device__ __forceinline__ float small_u32_to_float(uint32_t v) { return __uint_as_float(0x4B000000u | v) - 8388608.f; }
// Two f32 lanes in one 64-bit register, for the packed f32x2 arithmetic of sm_100 (IEEE per lane).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
// One 32-bit word of two bf16 = round-to-nearest-even of fma(d1, q, c) per lane, q = f - 2^23.
__device__ __forceinline__ uint32_t deq2(uint64_t f, uint64_t minus_magic, uint64_t d1, uint64_t c)
{
    uint64_t q, v;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(q) : "l"(f), "l"(minus_magic));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(v) : "l"(d1), "l"(q), "l"(c));
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// Eight weights (one 4-bit value in each byte of w0, w1) -> bf16, exactly as the reference decoder computes them
// in f32 (d1 * q - mm, crates/ferric-gguf/src/lib.rs:813-822) and then rounds to nearest even.  d1 * q is exact
// in f32 (<= 21 significant bits), so the fused multiply-add rounds once, like the separate multiply and subtract.
// A byte permute drops each value into the mantissa of 2^23 (0x4B000000 | q = 2^23 + q); subtracting 2^23 is exact.
__device__ __forceinline__ uint4 deq8(uint32_t w0, uint32_t w1, float d1, float mm)
{
    const uint64_t dd = pack_f32x2(d1, d1), cc = pack_f32x2(-mm, -mm), mg = pack_f32x2(-8388608.f, -8388608.f);
    auto word = [&](uint32_t w, int e) {
        return pack_f32x2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 + e)),
                          __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7651 + e)));
    };
    uint4 o;
    o.x = deq2(word(w0, 0), mg, dd, cc);
    o.y = deq2(word(w0, 2), mg, dd, cc);
    o.z = deq2(word(w1, 0), mg, dd, cc);
    o.w = deq2(word(w1, 2), mg, dd, cc);
    return o;
}

// Where K chunk j of super-block b goes in a ring of S stages of CH chunks: the stage, its wait parity, whether this
// chunk opens the stage (wait for it to be free) or closes it (announce it), and the chunk's A tile inside it.
template <int S, int CH>
struct GemmRingPos {
    int s, cc;
    uint32_t parity;
    __device__ __forceinline__ GemmRingPos(int b, int j)
    {
        const int e = (4 * b + j) / CH;
        cc = j % CH;
        s = e % S;
        parity = (((uint32_t)e / S) & 1u) ^ 1u;
    }
    __device__ __forceinline__ bool opens() const { return cc == 0; }
    __device__ __forceinline__ bool closes() const { return cc == CH - 1; }
    __device__ __forceinline__ uint32_t a_off() const { return (uint32_t)((s * CH + cc) * kGemmABytes); }
};

// ---------------------------------------------------------------- dequant stages
// One call per dequant warp: for every super-block, wait for its raw units, pull this warp's 16-row unit into
// registers, and for each of its four K chunks convert 16 rows x 64 weights to bf16, wait for a free A stage,
// store, and announce it.  Returns 0, or the code of the wait that ran out.
template <bool PAIR, bool Q5, int S, int CH>
__device__ __forceinline__ int dequant_loop_q4k(GemmBarriers* bar, uint8_t* a_stage, const uint8_t* raw_stage, int nblk,
                                                int tiles_here, int wq, int lane)
{
    // Q5: the Q5_K unit is the Q4_K unit plus a fifth-bit segment (lane 4g + t: qh[8t .. 8t+8) of rows g and g + 8); bit s
    // of qh[l] lifts value l of sub-block s by 16 (crates/ferric-gguf/src/lib.rs:690-716), the rest is Q4_K's arithmetic.
    constexpr int kUnitBytes = Q5 ? kQ5KUnit : kQ4KUnit;
    // ---------------- dequantise: warp = one 16-row unit (or eight rows of it), lane = (row g, 8-byte piece t)
    // The lane -> (g, t) map keeps both the 16-byte loads of the raw unit and the 16-byte stores into the
    // swizzled A tile free of bank conflicts: the two rows of a quarter-warp differ in bits 0 and 2.
    const int wd = wq;
    int fail = 0;
    const int t = lane & 3, qd = lane >> 3, g = ((lane >> 2) & 1) ? (qd ^ 5) : qd;
    const bool unit_ok = wd < tiles_here;
    const uint32_t arow_off = (uint32_t)(2 * wd * 1024 + g * 128);
    const uint32_t col_lo = (uint32_t)((t ^ g) << 4), col_hi = (uint32_t)(((4 + t) ^ g) << 4);
    for (int b = 0; b < nblk && !fail; b++) {
        const int rs = b % kGemmRawStages;
        if (!mbar_wait(&bar->raw_full[rs], ((uint32_t)b / kGemmRawStages) & 1u)) { fail = 4; break; }
        const uint8_t* u = raw_stage + rs * (8 * kUnitBytes) + wd * kUnitBytes;
        uint4 hdr[kGemmHalves], qs[kGemmHalves][2];
        uint2 q5[kGemmHalves];
        float d[kGemmHalves], dmin[kGemmHalves];
#pragma unroll
        for (int hh = 0; hh < kGemmHalves; hh++) {
            const int hi = hh;
            hdr[hh] = qs[hh][0] = qs[hh][1] = make_uint4(0, 0, 0, 0);
            q5[hh] = make_uint2(0, 0);
            if (unit_ok) {
                hdr[hh] = *reinterpret_cast<const uint4*>(u + 16 * (g + 8 * hi));
                qs[hh][0] = *reinterpret_cast<const uint4*>(u + 256 + 512 * (2 * hi) + 16 * (4 * g + t));
                qs[hh][1] = *reinterpret_cast<const uint4*>(u + 256 + 512 * (2 * hi + 1) + 16 * (4 * g + t));
                if (Q5) q5[hh] = *reinterpret_cast<const uint2*>(u + kQ5KOffQh + 16 * (4 * g + t) + 8 * hi);
            }
            d[hh] = __half2float(__ushort_as_half((unsigned short)(hdr[hh].x & 0xffffu)));
            dmin[hh] = __half2float(__ushort_as_half((unsigned short)(hdr[hh].x >> 16)));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar->raw_empty[rs]);   // the block now lives in registers
        // The four lanes of a row share its header: lane t works out (d*sc, dmin*m) of the two sub-blocks of
        // chunk t once, and every chunk fetches its pair from the lane that holds it.
        float my_d1a[kGemmHalves], my_mma[kGemmHalves], my_d1b[kGemmHalves], my_mmb[kGemmHalves];
#pragma unroll
        for (int hh = 0; hh < kGemmHalves; hh++) {
            uint32_t sc0, mn0, sc1, mn1;
            q4k_scale_min_dyn(hdr[hh], 2 * t, sc0, mn0);
            q4k_scale_min_dyn(hdr[hh], 2 * t + 1, sc1, mn1);
            my_d1a[hh] = __fmul_rn(d[hh], small_u32_to_float(sc0));
            my_mma[hh] = __fmul_rn(dmin[hh], small_u32_to_float(mn0));
            my_d1b[hh] = __fmul_rn(d[hh], small_u32_to_float(sc1));
            my_mmb[hh] = __fmul_rn(dmin[hh], small_u32_to_float(mn1));
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint4 lo[kGemmHalves], up[kGemmHalves];
            const int src = (lane & ~3) | j;
#pragma unroll
            for (int hh = 0; hh < kGemmHalves; hh++) {
                const float d1a = __shfl_sync(0xffffffffu, my_d1a[hh], src), mma = __shfl_sync(0xffffffffu, my_mma[hh], src);
                const float d1b = __shfl_sync(0xffffffffu, my_d1b[hh], src), mmb = __shfl_sync(0xffffffffu, my_mmb[hh], src);
                const uint4 q4 = qs[hh][j >> 1];
                const uint32_t w0 = (j & 1) ? q4.z : q4.x, w1 = (j & 1) ? q4.w : q4.y;
                uint32_t l0 = w0 & 0x0F0F0F0Fu, l1 = w1 & 0x0F0F0F0Fu, u0 = (w0 >> 4) & 0x0F0F0F0Fu, u1 = (w1 >> 4) & 0x0F0F0F0Fu;
                if (Q5) {   // sub-blocks 2j (low nibbles) and 2j + 1 (high nibbles)
                    l0 |= ((q5[hh].x >> (2 * j)) & 0x01010101u) << 4;
                    l1 |= ((q5[hh].y >> (2 * j)) & 0x01010101u) << 4;
                    u0 |= ((q5[hh].x >> (2 * j + 1)) & 0x01010101u) << 4;
                    u1 |= ((q5[hh].y >> (2 * j + 1)) & 0x01010101u) << 4;
                }
                lo[hh] = deq8(l0, l1, d1a, mma);
                up[hh] = deq8(u0, u1, d1b, mmb);
            }
            const GemmRingPos<S, CH> pos(b, j);
            const int s = pos.s;
            if (pos.opens() && !mbar_wait(&bar->a_empty[s], pos.parity)) { fail = 5; break; }
            uint8_t* arow = a_stage + pos.a_off() + arow_off;
#pragma unroll
            for (int hh = 0; hh < kGemmHalves; hh++) {
                *reinterpret_cast<uint4*>(arow + hh * 1024 + col_lo) = lo[hh];
                *reinterpret_cast<uint4*>(arow + hh * 1024 + col_hi) = up[hh];
            }
            if (pos.closes()) {
                fence_proxy_async();     // generic-proxy stores -> visible to the tensor core's async reads
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(cluster_addr(&bar->a_full[s], 0));
                    else mbar_arrive(&bar->a_full[s]);
                }
            }
        }
    }
    return fail;
}

// Four Q6_K weights (one 6-bit value in each byte of q) -> bf16 of t * (q - 32), t = d * scale, in the reference
// decoder's order (crates/ferric-gguf/src/lib.rs:721-746: (d * sc) * (q - 32)): q - 32 first (exact; +0 at q = 32),
// then the product (exact in f32: 18 x 6 bits, and with the decoder's sign of zero), then the rounding to bf16.
__device__ __forceinline__ uint2 deq4_q6(uint32_t q, float t)
{
    const uint64_t tt = pack_f32x2(t, t), mg = pack_f32x2(-8388640.f, -8388640.f);   // -(2^23 + 32)
    auto two = [&](int e) {
        const uint64_t f = pack_f32x2(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7650 + e)),
                                      __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7651 + e)));
        uint64_t qm, v;
        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(qm) : "l"(f), "l"(mg));
        asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(v) : "l"(tt), "l"(qm));
        float lo, hi;
        asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
        uint32_t r;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    };
    return make_uint2(two(0), two(2));
}

// Q6_K unit (layout.h): d pairs | int8 scales [16 rows][16] | ql: 4 segments (2 * half + c) | qh: 2 segments.
// Lane (g, t) holds, per row, ql words (c, h, is) = raw ql bytes [64h + 32c + 16is + 4t, +4) and qh words
// (h, is) = raw qh bytes [32h + 16is + 4t, +4).  K chunk j = (h, kp) = (j >> 1, j & 1) takes sub-blocks
// k = 2kp + c: nibble kp of the ql word, bits 2k..2k+1 of the qh word, chunk-local position 32c + 16is + 4t.
template <bool PAIR, int S, int CH>
__device__ __forceinline__ int dequant_loop_q6k(GemmBarriers* bar, uint8_t* a_stage, const uint8_t* raw_stage, int nblk,
                                                int tiles_here, int wq, int lane)
{
    const int wd = wq;
    int fail = 0;
    const int t = lane & 3, qd = lane >> 3, g = ((lane >> 2) & 1) ? (qd ^ 5) : qd;
    const bool unit_ok = wd < tiles_here;
    const uint32_t arow_off = (uint32_t)(2 * wd * 1024 + g * 128);
    for (int b = 0; b < nblk && !fail; b++) {
        const int rs = b % kGemmRawStages;
        if (!mbar_wait(&bar->raw_full[rs], ((uint32_t)b / kGemmRawStages) & 1u)) { fail = 4; break; }
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
        if (lane == 0) mbar_arrive(&bar->raw_empty[rs]);   // the block now lives in registers
        // Lane t works out d * scale for the four sub-blocks of chunk t (scale bytes 4t .. 4t+3 = word t of the
        // row's 16, byte 2c + is); every chunk fetches its four from the lane that holds them.
        float my_t[2][4];
#pragma unroll
        for (int hi = 0; hi < 2; hi++) {
            const float d = __half2float(__ushort_as_half((unsigned short)(hi ? (dpair >> 16) : (dpair & 0xffffu))));
            const uint32_t w = t == 0 ? sc[hi].x : (t == 1 ? sc[hi].y : (t == 2 ? sc[hi].z : sc[hi].w));
#pragma unroll
            for (int i = 0; i < 4; i++) my_t[hi][i] = __fmul_rn(d, (float)(int)(int8_t)(w >> (8 * i)));
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int h = j >> 1, kp = j & 1, src = (lane & ~3) | j;
            uint2 out[2][4];
#pragma unroll
            for (int hi = 0; hi < 2; hi++) {
#pragma unroll
                for (int c = 0; c < 2; c++) {
#pragma unroll
                    for (int is = 0; is < 2; is++) {
                        const float tv = __shfl_sync(0xffffffffu, my_t[hi][2 * c + is], src);
                        const uint4 qlv = ql[hi][c];
                        const uint32_t lw = (2 * h + is) == 0 ? qlv.x : ((2 * h + is) == 1 ? qlv.y : ((2 * h + is) == 2 ? qlv.z : qlv.w));
                        const uint32_t hw = (2 * h + is) == 0 ? qh[hi].x : ((2 * h + is) == 1 ? qh[hi].y : ((2 * h + is) == 2 ? qh[hi].z : qh[hi].w));
                        const uint32_t q = ((lw >> (4 * kp)) & 0x0F0F0F0Fu) | (((hw >> (2 * (2 * kp + c))) & 0x03030303u) << 4);
                        out[hi][2 * c + is] = deq4_q6(q, tv);
                    }
                }
            }
            const GemmRingPos<S, CH> pos(b, j);
            const int s = pos.s;
            if (pos.opens() && !mbar_wait(&bar->a_empty[s], pos.parity)) { fail = 5; break; }
            uint8_t* arow = a_stage + pos.a_off() + arow_off;
#pragma unroll
            for (int hi = 0; hi < 2; hi++)
#pragma unroll
                for (int i = 0; i < 4; i++)   // i = 2c + is: 16-byte column 2i + (t >> 1), half t & 1
                    *reinterpret_cast<uint2*>(arow + hi * 1024 + (((2 * i + (t >> 1)) ^ g) << 4) + 8 * (t & 1)) = out[hi][i];
            if (pos.closes()) {
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(cluster_addr(&bar->a_full[s], 0));
                    else mbar_arrive(&bar->a_full[s]);
                }
            }
        }
    }
    return fail;
}

// Q8_0 (crates/ferric-gguf/src/lib.rs:608-615: out = q * d): a stage holds [128 rows][256] int8 and [128][8] f16
// scales.  Thread = (row, 32-value block of the K chunk); q * d is exact in f32 (8 x 11 bits), then rounded to bf16.
template <bool PAIR, int S, int CH>
__device__ __forceinline__ int dequant_loop_q8_0(GemmBarriers* bar, uint8_t* a_stage, const uint8_t* raw_stage, int nb, int wq,
                                                 int lane)
{
    int fail = 0;
    const int td = 32 * wq + lane, r = td >> 1, half = td & 1;
    const uint32_t arow_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
    const uint64_t mg = pack_f32x2(-8388736.f, -8388736.f);   // -(2^23 + 128)
    for (int b = 0; b < nb && !fail; b++) {
        const int rs = b % kGemmRawStages;
        if (!mbar_wait(&bar->raw_full[rs], ((uint32_t)b / kGemmRawStages) & 1u)) { fail = 4; break; }
        const uint8_t* st = raw_stage + rs * gemm_raw_bytes(kGgmlQ8_0);
        uint4 qv[4][2];
        const uint4 dv = *reinterpret_cast<const uint4*>(st + kGemmQ8QsBytes + 16 * r);   // the row's 8 scales
#pragma unroll
        for (int j = 0; j < 4; j++) {
            qv[j][0] = *reinterpret_cast<const uint4*>(st + 256 * r + 64 * j + 32 * half);
            qv[j][1] = *reinterpret_cast<const uint4*>(st + 256 * r + 64 * j + 32 * half + 16);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar->raw_empty[rs]);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t dw = j == 0 ? dv.x : (j == 1 ? dv.y : (j == 2 ? dv.z : dv.w));
            const float d = __half2float(__ushort_as_half((unsigned short)(half ? (dw >> 16) : (dw & 0xffffu))));
            const uint64_t dd = pack_f32x2(d, d);
            uint4 out[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {   // 8 values -> one 16-byte column
                const uint32_t w0 = (i & 1) ? qv[j][i >> 1].z : qv[j][i >> 1].x, w1 = (i & 1) ? qv[j][i >> 1].w : qv[j][i >> 1].y;
                auto two = [&](uint32_t w, int e) {
                    // byte + 128 dropped into the mantissa of 2^23; subtracting 2^23 + 128 leaves the signed value exactly
                    const uint32_t u = w ^ 0x80808080u;
                    const uint64_t f = pack_f32x2(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650 + e)),
                                                  __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651 + e)));
                    uint64_t q, v;
                    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(q) : "l"(f), "l"(mg));
                    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(v) : "l"(q), "l"(dd));
                    float lo, hi;
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
                    uint32_t rr;
                    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(rr) : "f"(hi), "f"(lo));
                    return rr;
                };
                out[i] = make_uint4(two(w0, 0), two(w0, 2), two(w1, 0), two(w1, 2));
            }
            const GemmRingPos<S, CH> pos(b, j);
            const int s = pos.s;
            if (pos.opens() && !mbar_wait(&bar->a_empty[s], pos.parity)) { fail = 5; break; }
            uint8_t* arow = a_stage + pos.a_off() + arow_off;
#pragma unroll
            for (int i = 0; i < 4; i++) *reinterpret_cast<uint4*>(arow + (((4 * half + i) ^ (r & 7)) << 4)) = out[i];
            if (pos.closes()) {
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(cluster_addr(&bar->a_full[s], 0));
                    else mbar_arrive(&bar->a_full[s]);
                }
            }
        }
    }
    return fail;
}

// How a paired launch walks its tiles.  Pair tiles (256 weight rows x N_TILE activation rows) are numbered
// p = px + pairs_x * ny.  The first `full` of them are computed whole, one pair of CTAs each.  The rest -- the tiles
// that would make up a partly filled last wave -- are cut along K into `splits` pieces of `bps` super-blocks, each piece
// a pair of CTAs of its own that writes a partial tile to a workspace; a finish kernel adds the pieces in order.
struct GemmSplit {
    int pairs_x;     // pair tiles along the weight rows
    int full;        // tiles computed whole
    int splits;      // pieces per remaining tile (1 = none are cut)
    int bps;         // super-blocks per piece
};

template <uint32_t TY, int N_TILE, bool PAIR>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_q_bf16_kernel(const uint8_t* __restrict__ units, const __grid_constant__ CUtensorMap xmap,
                     const __grid_constant__ CUtensorMap ymap, const __grid_constant__ CUtensorMap wsmap,
                     const __grid_constant__ CUtensorMap q8map, const __grid_constant__ CUtensorMap q8dmap, GemmSplit split,
                     int tma_store, float* __restrict__ y, int rows, int nblk, int m, size_t ldy, int row_tiles16,
                     int* __restrict__ err)
{
    extern __shared__ uint8_t gemm_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* a_stage = smem;                                               // [S][CH][16384]
    constexpr bool kMerged = gemm_merged(N_TILE, PAIR);                    // one ring, two chunks per stage (see above)
    constexpr int kAStages = kMerged ? gemm_merged_stages(N_TILE) : kGemmStages, kCh = kMerged ? gemm_merged_chunks(N_TILE) : 1;
    constexpr int kBBytes = gemm_b_bytes(N_TILE, PAIR);
    constexpr int kBStages = kMerged ? kAStages * kCh : gemm_b_stages(TY, N_TILE, PAIR);   // B tiles held
    constexpr int kUnit = gemm_unit_bytes(TY), kRawBytes = gemm_raw_bytes(TY);
    constexpr int kNMma = N_TILE > 256 ? 256 : N_TILE;                     // activation rows per tcgen05.mma
    constexpr int kBoxRows = PAIR ? kNMma / 2 : kNMma;                     // of them, rows this CTA holds
    constexpr int kPeers = PAIR ? 2 : 1;
    uint8_t* b_stage = a_stage + kAStages * kCh * kGemmABytes;             // [kBStages][kBBytes]
    uint8_t* raw_stage = b_stage + kBStages * kBBytes;                     // [2][18432]
    GemmBarriers* bar = reinterpret_cast<GemmBarriers*>(raw_stage + kGemmRawStages * kRawBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;                   // rank 0 leads the pair
    // which tile, and which range of super-blocks of it
    int tile_x = blockIdx.x, tile_y = blockIdx.y, blk0 = 0, nb = nblk, piece = -1;
    if (PAIR) {
        const int item = blockIdx.x >> 1;
        int p = item;
        if (item >= split.full) {
            const int e = item - split.full;
            p = split.full + e / split.splits;
            piece = e;                                                     // index of this partial tile in the workspace
            blk0 = (e % split.splits) * split.bps;
            nb = max(0, min(nblk, blk0 + split.bps) - blk0);
        }
        tile_x = 2 * (p % split.pairs_x) + (int)rank;
        tile_y = p / split.pairs_x;
    }
    const int row0 = tile_x * kGemmRows, n0 = tile_y * N_TILE;
    const int rt0 = tile_x * 8;                                            // first 16-row tile of this CTA
    const int tiles_here = max(0, min(8, row_tiles16 - rt0));              // 0: padding CTA of an odd pair
    const int nchunks = nb * 4;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kGemmRawStages; i++) {
            mbar_init(&bar->raw_full[i], 1);
            mbar_init(&bar->raw_empty[i], kGemmDeqWarps);
        }
        for (int i = 0; i < kAStages; i++) {
            mbar_init(&bar->a_full[i], kGemmDeqWarps * kPeers + (kMerged ? kPeers : 0));   // in a pair only the leader's is used
            mbar_init(&bar->a_empty[i], 1);
        }
        for (int i = 0; i < kBStages; i++) {
            mbar_init(&bar->b_full[i], kPeers);
            mbar_init(&bar->b_empty[i], 1);
        }
        mbar_init(&bar->acc_full, 1);
        bar->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // tensor memory for the 128 x N_TILE f32 accumulator (in a pair: one warp of each CTA)
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_base)),
                         "n"(N_TILE)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_base)),
                         "n"(N_TILE)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_acc = bar->tmem_base;
    int fail = 0;

    if (warp == 0) {
        // ---------------- weight producer: raw quant units of one super-block per stage
        if (lane == 0) {
            for (int b = 0; b < nb; b++) {
                const int rs = b % kGemmRawStages;
                if (!mbar_wait(&bar->raw_empty[rs], (((uint32_t)b / kGemmRawStages) & 1u) ^ 1u)) { fail = 1; break; }
                if (TY == kGgmlQ8_0) {   // two boxes; rows and columns past the matrix read as zeros
                    mbar_expect_tx(&bar->raw_full[rs], (uint32_t)kRawBytes);
                    tma_load_2d(raw_stage + rs * kRawBytes, &q8map, 256 * (blk0 + b), row0, &bar->raw_full[rs]);
                    tma_load_2d(raw_stage + rs * kRawBytes + kGemmQ8QsBytes, &q8dmap, 8 * (blk0 + b), row0, &bar->raw_full[rs]);
                    continue;
                }
                mbar_expect_tx(&bar->raw_full[rs], (uint32_t)(tiles_here * kUnit));
                for (int t = 0; t < tiles_here; t++)
                    bulk_g2s(raw_stage + rs * kRawBytes + t * kUnit, units + ((size_t)(rt0 + t) * nblk + blk0 + b) * kUnit, kUnit,
                             &bar->raw_full[rs]);
            }
        }
    } else if (warp == 2) {
        // ---------------- activation producer: one [64 k x N_TILE rows] bf16 tile per stage
        if (lane == 0 && kMerged) {
            for (int e = 0; e < nchunks / kCh; e++) {
                const int s = e % kAStages;
                if (!mbar_wait(&bar->a_empty[s], (((uint32_t)e / kAStages) & 1u) ^ 1u)) { fail = 2; break; }
                if (PAIR) {
                    // each CTA fetches its half of every 256-row operand; the bytes of both are counted by the leader
                    const uint32_t full = cluster_addr(&bar->a_full[s], 0);
                    mbar_expect_tx_cluster(full, (uint32_t)(kCh * kBBytes));
#pragma unroll
                    for (int cc = 0; cc < kCh; cc++)
#pragma unroll
                        for (int h = 0; h < N_TILE / kNMma; h++)
                            tma_load_2d_pair(b_stage + (s * kCh + cc) * kBBytes + h * kBoxRows * 128, &xmap,
                                             (4 * blk0 + kCh * e + cc) * kGemmChunkK, n0 + h * kNMma + (int)rank * kBoxRows, full);
                } else {
                    mbar_expect_tx(&bar->a_full[s], (uint32_t)(kCh * kBBytes));
#pragma unroll
                    for (int cc = 0; cc < kCh; cc++)
                        tma_load_2d(b_stage + (s * kCh + cc) * kBBytes, &xmap, (kCh * e + cc) * kGemmChunkK, n0, &bar->a_full[s]);
                }
            }
        } else if (lane == 0) {
            for (int c = 0; c < nchunks; c++) {
                const int s = c % kBStages;
                if (!mbar_wait(&bar->b_empty[s], (((uint32_t)c / kBStages) & 1u) ^ 1u)) { fail = 2; break; }
                if (PAIR) {
                    // each CTA fetches its half of every 256-row operand; the bytes of both are counted by the leader
                    const uint32_t full = cluster_addr(&bar->b_full[s], 0);
                    mbar_expect_tx_cluster(full, (uint32_t)kBBytes);
#pragma unroll
                    for (int h = 0; h < N_TILE / kNMma; h++)
                        tma_load_2d_pair(b_stage + s * kBBytes + h * kBoxRows * 128, &xmap, (4 * blk0 + c) * kGemmChunkK,
                                         n0 + h * kNMma + (int)rank * kBoxRows, full);
                } else {
                    mbar_expect_tx(&bar->b_full[s], (uint32_t)kBBytes);
#pragma unroll
                    for (int h = 0; h < N_TILE / kNMma; h++)   // one box of at most 256 activation rows each
                        tma_load_2d(b_stage + s * kBBytes + h * kNMma * 128, &xmap, c * kGemmChunkK, n0 + h * kNMma, &bar->b_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0 && kMerged) {
            if (rank == 0) {
                constexpr uint32_t idesc = umma_idesc_bf16(kGemmRows * kPeers, kNMma);
                for (int e = 0; e < nchunks / kCh; e++) {
                    const int s = e % kAStages;
                    if (!mbar_wait(&bar->a_full[s], ((uint32_t)e / kAStages) & 1u)) { fail = 3; break; }
                    tc_fence_after();
#pragma unroll
                    for (int cc = 0; cc < kCh; cc++) {
                        const uint32_t a0 = smem_u32(a_stage + (s * kCh + cc) * kGemmABytes), b0 = smem_u32(b_stage + (s * kCh + cc) * kBBytes);
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++)
#pragma unroll
                            for (int h = 0; h < N_TILE / kNMma; h++) {
                                const uint64_t ad = umma_desc_sw128(a0 + 32 * k4), bd = umma_desc_sw128(b0 + h * kBoxRows * 128 + 32 * k4);
                                if (PAIR) umma_bf16_pair(tmem_acc + h * kNMma, ad, bd, idesc, (e | cc | k4) ? 1u : 0u);
                                else umma_bf16(tmem_acc + h * kNMma, ad, bd, idesc, (e | cc | k4) ? 1u : 0u);
                            }
                    }
                    // one commit frees the stage (in both CTAs of a pair) once the MMAs above have read it
                    if (PAIR) umma_commit_pair(&bar->a_empty[s]);
                    else umma_commit(&bar->a_empty[s]);
                }
                if (!fail) {
                    if (PAIR) umma_commit_pair(&bar->acc_full);
                    else umma_commit(&bar->acc_full);
                }
            }
        } else if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(kGemmRows * kPeers, kNMma);
            for (int c = 0; c < nchunks; c++) {
                const int sa = c % kGemmStages, sb = c % kBStages;
                if (!mbar_wait(&bar->a_full[sa], ((uint32_t)c / kGemmStages) & 1u) ||
                    !mbar_wait(&bar->b_full[sb], ((uint32_t)c / kBStages) & 1u)) { fail = 3; break; }
                tc_fence_after();
                const uint32_t a0 = smem_u32(a_stage + sa * kGemmABytes), b0 = smem_u32(b_stage + sb * kBBytes);
#pragma unroll
                for (int k4 = 0; k4 < 4; k4++)
#pragma unroll
                    for (int h = 0; h < N_TILE / kNMma; h++) {
                        const uint64_t ad = umma_desc_sw128(a0 + 32 * k4), bd = umma_desc_sw128(b0 + h * kBoxRows * 128 + 32 * k4);
                        if (PAIR) umma_bf16_pair(tmem_acc + h * kNMma, ad, bd, idesc, (c | k4) ? 1u : 0u);
                        else umma_bf16(tmem_acc + h * kNMma, ad, bd, idesc, (c | k4) ? 1u : 0u);
                    }
                // each commit frees its stage (in both CTAs of a pair) once the MMAs above have read it
                if (PAIR) {
                    umma_commit_pair(&bar->a_empty[sa]);
                    umma_commit_pair(&bar->b_empty[sb]);
                } else {
                    umma_commit(&bar->a_empty[sa]);
                    umma_commit(&bar->b_empty[sb]);
                }
            }
            if (!fail) {
                if (PAIR) umma_commit_pair(&bar->acc_full);
                else umma_commit(&bar->acc_full);
            }
        }
    } else {
        // ---------------- dequantise (per quant type, above), then the epilogue
        const int wq = warp - kGemmFirstDeqWarp;
        if (TY == kGgmlQ4K) fail = dequant_loop_q4k<PAIR, false, kAStages, kCh>(bar, a_stage, raw_stage, nb, tiles_here, wq, lane);
        else if (TY == kGgmlQ5K) fail = dequant_loop_q4k<PAIR, true, kAStages, kCh>(bar, a_stage, raw_stage, nb, tiles_here, wq, lane);
        else if (TY == kGgmlQ6K) fail = dequant_loop_q6k<PAIR, kAStages, kCh>(bar, a_stage, raw_stage, nb, tiles_here, wq, lane);
        else fail = dequant_loop_q8_0<PAIR, kAStages, kCh>(bar, a_stage, raw_stage, nb, wq, lane);
        // ---------------- epilogue.  All dequant warps first agree that nobody gave up (the staged path below
        // synchronises them with named barriers, which must not be entered by only some of them).
        if (fail) atomicExch(&bar->abort, fail);
        named_bar_sync(1, 32 * kGemmDeqWarps);
        if (*reinterpret_cast<volatile int*>(&bar->abort) == 0 && wq < 8 && !mbar_wait(&bar->acc_full, 0)) {
            fail = 6;
            atomicExch(&bar->abort, fail);
        }
        named_bar_sync(1, 32 * kGemmDeqWarps);
        if (*reinterpret_cast<volatile int*>(&bar->abort) == 0 && wq < 8) {
            tc_fence_after();
            // A warp may read TMEM lanes 32*(warp%4) .. +32; lane = weight row, column = activation row.
            const int q = warp & 3, grp = wq >> 2, wrow = row0 + 32 * q + lane;
            if (tma_store) {
                // Two groups of four warps take alternate 32-column slabs: TMEM -> registers -> a [32][128] f32
                // staging tile (two per group, in the idle activation ring) -> one TMA store per slab, which
                // clips rows past `rows` and activation rows past `m`.
                float* stage0 = reinterpret_cast<float*>(b_stage + grp * 2 * kGemmStoreBytes);
                const bool elected = (wq & 3) == 0 && lane == 0;
                int it = 0;
#pragma unroll 1
                for (int c0 = 32 * grp; c0 < N_TILE; c0 += 64, it++) {
                    if (n0 + c0 >= m) break;                       // uniform over the group
                    float* stg = stage0 + (it & 1) * (kGemmStoreBytes / 4);
                    if (elected) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // tile (it - 2) has been read
                    named_bar_sync(2 + grp, 128);
                    uint32_t v[32];
                    tmem_ld_32(tmem_acc + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
#pragma unroll
                    for (int jj = 0; jj < 32; jj++) stg[jj * 128 + 32 * q + lane] = __uint_as_float(v[jj]);
                    fence_proxy_async();
                    named_bar_sync(2 + grp, 128);
                    if (elected && row0 < rows) {
                        if (piece < 0)   // a whole tile: straight into y
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&ymap),
                                         "r"(row0), "r"(n0 + c0), "r"(smem_u32(stg))
                                         : "memory");
                        else             // a K piece: into partial tile `piece` of the workspace, [N_TILE][256] f32
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&wsmap),
                                         "r"((int)rank * kGemmRows), "r"(piece * N_TILE + c0), "r"(smem_u32(stg))
                                         : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
                if (elected) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            } else if (wq < 4) {
#pragma unroll 1
                for (int c0 = 0; c0 < N_TILE; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32(tmem_acc + ((uint32_t)(32 * q) << 16) + (uint32_t)c0, v);
                    if (wrow < rows) {
#pragma unroll
                        for (int jj = 0; jj < 32; jj++) {
                            const int batch = n0 + c0 + jj;
                            if (batch < m) y[(size_t)batch * ldy + wrow] = __uint_as_float(v[jj]);
                        }
                    }
                }
            }
        }
    }
    if (fail) {
        atomicExch(&bar->abort, fail);
        if (err) atomicExch(err, fail);
    }
    tc_fence_before();
    __syncthreads();
    if (bar->abort) {
        // something never arrived: give copies still in flight time to land before the CTA's memory goes away
        for (int i = 0; i < 200; i++) __nanosleep(1000);
        __syncthreads();
    }
    // In a pair neither CTA may leave, or give its tensor memory back, while the other can still signal its barriers
    // or the leader's MMAs can still touch its shared and tensor memory.
    if (PAIR) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "n"(N_TILE) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "n"(N_TILE) : "memory");
    }
}

// Adds the K pieces of the cut tiles, in piece order, into y.  One block per (cut tile, activation row of it), one
// thread per weight row of the 256-row pair tile.
template <int N_TILE>
__global__ void __launch_bounds__(256)
gemm_finish_kernel(const float* __restrict__ ws, GemmSplit split, float* __restrict__ y, size_t ldy, int rows, int m)
{
    const int e_tile = blockIdx.x / N_TILE, c = blockIdx.x % N_TILE, r = threadIdx.x;
    const int p = split.full + e_tile, row = (p % split.pairs_x) * 2 * kGemmRows + r, act = (p / split.pairs_x) * N_TILE + c;
    if (row >= rows || act >= m) return;
    float sum = 0.0f;
    for (int s = 0; s < split.splits; s++) sum += ws[((size_t)(e_tile * split.splits + s) * N_TILE + c) * (2 * kGemmRows) + r];
    y[(size_t)act * ldy + row] = sum;
}

// ---------------------------------------------------------------- host side
// Set by a CTA whose bounded wait ran out (the code says which role gave up); read by gemm_status().
static __device__ int g_gemm_status = 0;

// Device address of the status word on the current device (nullptr if the lookup fails: kernels then skip reporting).
int* gemm_status_word()
{
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_gemm_status) != cudaSuccess) return nullptr;
    return p;
}

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn()
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

template <uint32_t TY, int N_TILE, bool PAIR>
int32_t launch_gemm_tile(cudaStream_t st, const DeviceWeights& w, const CUtensorMap& map, const CUtensorMap& ymap,
                         const CUtensorMap& wsmap, const CUtensorMap* q8maps, const GemmSplit& split, int tma_store, size_t m,
                         float* y, size_t ldy)
{
    static bool attr_done[64] = {};
    int dev = 0;
    FERRIC_CUDA_TRY(cudaGetDevice(&dev));
    constexpr int smem = gemm_smem_bytes(TY, N_TILE, PAIR);
    if (dev < 64 && !attr_done[dev]) {
        FERRIC_CUDA_TRY(cudaFuncSetAttribute(gemm_q_bf16_kernel<TY, N_TILE, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_done[dev] = true;
    }
    int* err = nullptr;
    FERRIC_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&err), g_gemm_status));
    const unsigned n_tiles = (unsigned)((m + N_TILE - 1) / N_TILE);
    unsigned gx = (unsigned)((w.rows + kGemmRows - 1) / kGemmRows);
    cudaLaunchConfig_t cfg = {};
    if (PAIR) {
        // one pair of CTAs per work item: the whole tiles, then the K pieces of the cut ones (an odd row-tile count
        // leaves a padding CTA that multiplies zeros and stores nothing)
        const unsigned tiles = (unsigned)split.pairs_x * n_tiles;
        const unsigned items = (unsigned)split.full + (tiles - (unsigned)split.full) * (unsigned)split.splits;
        cfg.gridDim = dim3(2 * items, 1);
    } else {
        cfg.gridDim = dim3(gx, n_tiles);
    }
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FERRIC_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_q_bf16_kernel<TY, N_TILE, PAIR>, (const uint8_t*)w.units, map, ymap, wsmap, q8maps[0],
                                       q8maps[1], split, tma_store, y, (int)w.rows, (int)w.nblk, (int)m, ldy, (int)w.row_tiles(), err));
    return kOk;
}

// FERRIC_CUDA_GEMM_PAIR=0 keeps every tile on a single CTA (for comparison runs).
bool gemm_pair_enabled()
{
    static const bool on = [] {
        const char* e = getenv("FERRIC_CUDA_GEMM_PAIR");
        return !(e && e[0] == '0');
    }();
    return on;
}
}  // namespace

template <uint32_t TY>
static int32_t launch_gemm_ty(cudaStream_t st, const DeviceWeights& w, const CUtensorMap& map, const CUtensorMap& ymap,
                              const CUtensorMap& wsmap, const CUtensorMap* q8maps, const GemmSplit& split, int tma_store, size_t m,
                              float* y, size_t ldy, int n_tile, bool pair)
{
    if (n_tile == 128) return launch_gemm_tile<TY, 128, false>(st, w, map, ymap, wsmap, q8maps, split, tma_store, m, y, ldy);
    if (n_tile == 256) return launch_gemm_tile<TY, 256, false>(st, w, map, ymap, wsmap, q8maps, split, tma_store, m, y, ldy);
    if (pair) return launch_gemm_tile<TY, 512, true>(st, w, map, ymap, wsmap, q8maps, split, tma_store, m, y, ldy);
    if constexpr (TY != kGgmlQ8_0) return launch_gemm_tile<TY, 512, false>(st, w, map, ymap, wsmap, q8maps, split, tma_store, m, y, ldy);
    return kUnsupported;   // not reached: Q8_0 takes 256-wide tiles when pairing is off
}

// The cut: with P pair tiles on `slots` pair slots, the P mod slots tiles of the last, partly filled wave are each cut into
// as many K pieces as fill that wave (fewer tiles than slots: every tile is cut).  FERRIC_CUDA_GEMM_SPLIT=0 disables it.
GemmSplit gemm_split_plan(const DeviceWeights& w, size_t m, int n_tile, int sm_count)
{
    static const bool enabled = [] {
        const char* e = getenv("FERRIC_CUDA_GEMM_SPLIT");
        return !(e && e[0] == '0');
    }();
    GemmSplit sp;
    sp.pairs_x = (int)((w.rows + 2 * kGemmRows - 1) / (2 * kGemmRows));
    const int tiles = sp.pairs_x * (int)((m + n_tile - 1) / n_tile), slots = sm_count / 2 > 0 ? sm_count / 2 : 1;
    sp.full = tiles;
    sp.splits = 1;
    sp.bps = (int)w.nblk;
    const int excess = tiles % slots;
    if (!enabled || excess == 0) return sp;
    int want = slots / excess;                            // pieces per cut tile that fill the last wave
    if (want > (int)w.nblk / 2) want = (int)w.nblk / 2;   // at least two super-blocks per piece
    if (want > 16) want = 16;
    if (want < 2) return sp;
    sp.bps = ((int)w.nblk + want - 1) / want;
    sp.splits = ((int)w.nblk + sp.bps - 1) / sp.bps;      // every piece is non-empty
    sp.full = tiles - excess;
    return sp;
}

size_t gemm_workspace_bytes(const DeviceWeights& w, size_t m, int sm_count)
{
    if (m <= 256 || !gemm_pair_enabled()) return 0;
    DeviceWeights wl = w;
    if (w.q8_qs) wl.nblk = w.cols / 256;   // Q8_0: the kernel walks K in groups of 256
    const GemmSplit sp = gemm_split_plan(wl, m, 512, sm_count);
    if (sp.splits <= 1) return 0;
    const size_t tiles = (size_t)sp.pairs_x * ((m + 511) / 512);
    return (tiles - (size_t)sp.full) * (size_t)sp.splits * 512 * (2 * kGemmRows) * sizeof(float);
}

int32_t launch_gemm_bf16(cudaStream_t st, uint32_t ty, const DeviceWeights& w_in, const uint16_t* x_bf16, size_t m, size_t ldx,
                         float* y, size_t ldy, void* workspace, int sm_count)
{
    if (ty != kGgmlQ4K && ty != kGgmlQ5K && ty != kGgmlQ6K && ty != kGgmlQ8_0) return kUnsupported;
    if (m == 0 || w_in.rows == 0 || w_in.nblk == 0) return kOk;
    DeviceWeights w = w_in;
    if (ty == kGgmlQ8_0) {
        if (w.cols % 256 != 0) {
            set_last_error("the Q8_0 tensor-core product needs a multiple of 256 columns, matrix has %zu", w.cols);
            return kUnsupported;
        }
        w.nblk = w.cols / 256;   // the kernel walks K in groups of 256 for every format
    }
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (ldx * 2) % 16 != 0) {
        set_last_error("bf16 activations must be 16-byte aligned with a row stride that is a multiple of 8 elements");
        return kErrInvalidArg;
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) {
        set_last_error("the CUDA driver does not export cuTensorMapEncodeTiled");
        return kErrCuda;
    }
    int n_tile = m <= 128 ? 128 : (m <= 256 ? 256 : 512);
    if (ty == kGgmlQ8_0 && !gemm_pair_enabled() && n_tile == 512) n_tile = 256;   // its stage leaves room for 512 only in a pair
    const bool pair = n_tile == 512 && gemm_pair_enabled();   // two CTAs share each activation tile
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)w.cols, (cuuint64_t)m};
    const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kGemmChunkK, (cuuint32_t)(pair ? 128 : (n_tile > 256 ? 256 : n_tile))};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(x_bf16), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed with code %d", (int)r);
        return kErrCuda;
    }
    // The result leaves through TMA stores of [32 activation rows][128 weight rows] f32 tiles when y allows it
    // (16-byte aligned base and row pitch); otherwise the epilogue stores element-wise.
    CUtensorMap ymap;
    memset(&ymap, 0, sizeof(ymap));
    int tma_store = 0;
    if ((reinterpret_cast<uintptr_t>(y) & 15) == 0 && (ldy * 4) % 16 == 0) {
        const cuuint64_t ydims[2] = {(cuuint64_t)w.rows, (cuuint64_t)m};
        const cuuint64_t ystrides[1] = {(cuuint64_t)ldy * 4};
        const cuuint32_t ybox[2] = {(cuuint32_t)kGemmRows, 32};
        r = enc(&ymap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, y, ydims, ystrides, ybox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            set_last_error("cuTensorMapEncodeTiled (result) failed with code %d", (int)r);
            return kErrCuda;
        }
        tma_store = 1;
    }
    // The K pieces of cut tiles go to the workspace as partial tiles [piece][512 activation rows][256 weight rows].
    GemmSplit split = gemm_split_plan(w, m, n_tile, sm_count);
    if (!pair || !tma_store || !workspace) {
        split.full = split.pairs_x * (int)((m + n_tile - 1) / n_tile);
        split.splits = 1;
        split.bps = (int)w.nblk;
    }
    CUtensorMap wsmap;
    memset(&wsmap, 0, sizeof(wsmap));
    const size_t cut_tiles = (size_t)split.pairs_x * ((m + n_tile - 1) / n_tile) - (size_t)split.full;
    if (split.splits > 1) {
        const cuuint64_t wdims[2] = {(cuuint64_t)(2 * kGemmRows), (cuuint64_t)(cut_tiles * split.splits * n_tile)};
        const cuuint64_t wstrides[1] = {(cuuint64_t)(2 * kGemmRows) * 4};
        const cuuint32_t wbox[2] = {(cuuint32_t)kGemmRows, 32};
        r = enc(&wsmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, workspace, wdims, wstrides, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            set_last_error("cuTensorMapEncodeTiled (workspace) failed with code %d", (int)r);
            return kErrCuda;
        }
    }
    CUtensorMap q8maps[2];
    memset(q8maps, 0, sizeof(q8maps));
    if (ty == kGgmlQ8_0) {
        const cuuint64_t qdims[2] = {(cuuint64_t)w.cols, (cuuint64_t)w.rows}, qstr[1] = {(cuuint64_t)w.cols};
        const cuuint32_t qbox[2] = {256, (cuuint32_t)kGemmRows};
        r = enc(&q8maps[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w.q8_qs, qdims, qstr, qbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        const cuuint64_t ddims[2] = {(cuuint64_t)(w.cols / 32), (cuuint64_t)w.rows}, dstr[1] = {(cuuint64_t)(w.cols / 32) * 2};
        const cuuint32_t dbox[2] = {8, (cuuint32_t)kGemmRows};
        if (r == CUDA_SUCCESS)
            r = enc(&q8maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w.q8_d, ddims, dstr, dbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            set_last_error("cuTensorMapEncodeTiled (Q8_0 planes) failed with code %d", (int)r);
            return kErrCuda;
        }
    }
    int32_t rc = ty == kGgmlQ4K   ? launch_gemm_ty<kGgmlQ4K>(st, w, map, ymap, wsmap, q8maps, split, tma_store, m, y, ldy, n_tile, pair)
                 : ty == kGgmlQ5K ? launch_gemm_ty<kGgmlQ5K>(st, w, map, ymap, wsmap, q8maps, split, tma_store, m, y, ldy, n_tile, pair)
                 : ty == kGgmlQ6K ? launch_gemm_ty<kGgmlQ6K>(st, w, map, ymap, wsmap, q8maps, split, tma_store, m, y, ldy, n_tile, pair)
                                  : launch_gemm_ty<kGgmlQ8_0>(st, w, map, ymap, wsmap, q8maps, split, tma_store, m, y, ldy, n_tile, pair);
    if (rc != kOk || split.splits <= 1) return rc;
    gemm_finish_kernel<512><<<(unsigned)(cut_tiles * 512), 256, 0, st>>>(reinterpret_cast<const float*>(workspace), split, y, ldy,
                                                                        (int)w.rows, (int)m);
    FERRIC_CUDA_TRY(cudaGetLastError());
    return kOk;
}

// Synchronises the stream, returns the code of the first bounded wait that ran out (0 = none) and clears it.
int32_t gemm_status(cudaStream_t st, int* code)
{
    FERRIC_CUDA_TRY(cudaStreamSynchronize(st));
    int v = 0, zero = 0;
    FERRIC_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)));
    if (v) FERRIC_CUDA_TRY(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)));
    *code = v;
    return kOk;
}

}  // namespace ferric
