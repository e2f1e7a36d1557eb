// Device weight layout ("T16") and fragment maps for the packed-quant GEMV kernels.
//
// The reference re-packs GGUF block bytes on upload so its kernels read aligned u32 words
// (crates/ferric-tensor/src/dtype.rs:1388-1420 Q4_K, :1147-1166 Q6_K, :1270-1286 Q8_0).  This
// backend re-packs too, for a different machine: weights are grouped into *units* of 16 output
// rows x one 256-weight super-block, and inside a unit the bytes are permuted so that each warp
// load is one contiguous, fully coalesced 512-byte run of 128-bit words and every lane receives
// exactly the bytes its tensor-core fragment needs.  Total bytes are unchanged: 144 B (Q4_K) or
// 210 B (Q6_K) per 256 weights.
//
// Everything here is plain integer arithmetic shared by the device kernels and by a host-side
// emulation test, so the index maps can be verified without a GPU.
//
// Lane naming follows the mma.sync fragment layouts: lane = 4*g + t, g = 0..7, t = 0..3.
// Integer m16n8k32 (8-bit operands):
//   A regs {a0,a1,a2,a3} = (row g, k 4t..4t+3), (row g+8, k 4t..4t+3), (row g, k 16+4t..), (row g+8, k 16+4t..)
//   B regs {b0,b1}       = (k 4t..4t+3, col g), (k 16+4t..16+4t+3, col g)        byte j of a reg = k + j
//   C regs {c0..c3}      = (row g, cols 2t, 2t+1), (row g+8, cols 2t, 2t+1)
// m16n8k16 (8-bit) is the first half of that: A {a0,a1}, B {b0}.
// The k index is a summation index, so any permutation is legal as long as A and B agree.
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define FERRIC_HD __host__ __device__ __forceinline__
#else
#define FERRIC_HD inline
#endif

namespace ferric {

constexpr int kTileRows = 16;

// ---------------------------------------------------------------- Q4_K (ggml type 12)
// Raw block (crates/ferric-gguf/src/lib.rs:793-825): [f16 d][f16 dmin][scales 12][qs 128] = 144 B.
// qs holds four 32-byte groups; group p carries sub-block 2p in its low nibbles and 2p+1 in its
// high nibbles.  Unit (2304 B): hdr[16 rows][16 B] | 4 segments of 512 B.  Segment 2*(row>>3) + X
// (X = 0,1) holds groups 2X and 2X+1; lane 4*(row&7) + t owns 16 bytes: bytes [8t, 8t+8) of group
// 2X, then bytes [8t, 8t+8) of group 2X+1 -- i.e. eight weights of each of four sub-blocks.
constexpr int kQ4KBlock = 144;
constexpr int kQ4KUnit = 16 * kQ4KBlock;  // 2304
constexpr int kQ4KSteps = 10;             // 8 sub-block steps + sub-block sums + block scale

FERRIC_HD uint32_t q4k_unit_offset(int r, int byte)
{
    if (byte < 16) return (uint32_t)(r * 16 + byte);
    int beta = byte - 16;
    int g = r & 7, hi = r >> 3, p = beta >> 5, t = (beta >> 3) & 3, j = beta & 7, X = p >> 1;
    return (uint32_t)(256 + 512 * (2 * hi + X) + 16 * (4 * g + t) + 8 * (p & 1) + j);
}
// Weight (0..255 inside the super-block) that lane t supplies as byte i (0..7: b0 bytes 0..3, then
// b1 bytes 0..3) of sub-block step s (0..7).
FERRIC_HD int q4k_frag_weight(int s, int t, int i) { return 32 * s + 8 * t + i; }

// ---------------------------------------------------------------- Q5_K (ggml type 13)
// Raw block (crates/ferric-gguf/src/lib.rs:690-716): [f16 d][f16 dmin][scales 12][qh 32][qs 128] = 176 B: Q4_K with a
// fifth bit -- bit j of qh[l] belongs to value l of sub-block j.  Unit (2816 B): the Q4_K unit of the header and the
// nibbles, followed by one 512-byte segment of fifth bits in which lane 4*(row&7) + t owns 16 bytes: qh[8t, 8t+8) of
// row (row&7), then qh[8t, 8t+8) of row (row&7) + 8 -- the bits of exactly the eight weights per sub-block whose
// nibbles the lane holds.
constexpr int kQ5KBlock = 176;
constexpr int kQ5KUnit = 16 * kQ5KBlock;  // 2816
constexpr int kQ5KOffQh = kQ4KUnit;       // 2304

FERRIC_HD uint32_t q5k_unit_offset(int r, int byte)
{
    if (byte < 16) return (uint32_t)(r * 16 + byte);
    if (byte < 48) {
        int j = byte - 16, g = r & 7, hi = r >> 3;
        return (uint32_t)(kQ5KOffQh + 16 * (4 * g + (j >> 3)) + 8 * hi + (j & 7));
    }
    return q4k_unit_offset(r, byte - 32);   // the 128 quant bytes sit where Q4_K has them
}

// ---------------------------------------------------------------- Q6_K (ggml type 14)
// Raw block (crates/ferric-gguf/src/lib.rs:721-746): [ql 128][qh 64][i8 scales 16][f16 d] = 210 B.
// Sub-block sb = 8h + 2k + is (16 weights: 128h + 32k + 16is + j) takes its low 4 bits from
// ql[64h + 32(k&1) + 16is + j] (low nibble for k < 2, high nibble otherwise) and its high 2 bits
// from bits 2k..2k+1 of qh[32h + 16is + j].
// Unit (3360 B):
//   [   0,   32)  dpair[8]  u32: d(row g) | d(row g+8) << 16
//   [  32,  288)  sc[16 rows][16 B]: the raw int8 scales
//   [ 288, 2336)  ql: 4 segments of 512 B, segment 2*(row>>3) + c; lane 4g+t owns 4 words,
//                 word wi = 2h + is = raw ql bytes [64h + 32c + 16is + 4t, +4)
//   [2336, 3360)  qh: 2 segments of 512 B, segment row>>3; lane 4g+t owns 4 words,
//                 word wi = 2h + is = raw qh bytes [32h + 16is + 4t, +4)
constexpr int kQ6KBlock = 210;
constexpr int kQ6KUnit = 16 * kQ6KBlock;  // 3360
constexpr int kQ6KSteps = 10;             // 8 double sub-block steps + sub-block sums + block scale
constexpr int kQ6KOffSc = 32, kQ6KOffQl = 288, kQ6KOffQh = 2336;

FERRIC_HD uint32_t q6k_unit_offset(int r, int byte)
{
    int g = r & 7, hi = r >> 3;
    if (byte < 128) {
        int h = byte >> 6, c = (byte >> 5) & 1, is = (byte >> 4) & 1, t = (byte >> 2) & 3, jj = byte & 3;
        return (uint32_t)(kQ6KOffQl + 512 * (2 * hi + c) + 16 * (4 * g + t) + 4 * (2 * h + is) + jj);
    }
    if (byte < 192) {
        int b = byte - 128, h = b >> 5, is = (b >> 4) & 1, t = (b >> 2) & 3, jj = b & 3;
        return (uint32_t)(kQ6KOffQh + 512 * hi + 16 * (4 * g + t) + 4 * (2 * h + is) + jj);
    }
    if (byte < 208) return (uint32_t)(kQ6KOffSc + 16 * r + (byte - 192));
    return (uint32_t)(4 * g + 2 * hi + (byte - 208));
}
// Weight that lane t supplies as byte i (0..3) of sub-block sb (0..15).
FERRIC_HD int q6k_frag_weight(int sb, int t, int i) { return 16 * sb + 4 * t + i; }

// ---------------------------------------------------------------- Q8_0 (ggml type 8)
// Raw block (crates/ferric-gguf/src/lib.rs:608-615): [f16 d][i8 qs 32] = 34 B, 2-byte aligned.
// Device layout: two planes, qs[rows][cols] int8 (16-byte aligned rows) and d[rows][cols/32] f16.
constexpr int kQ8Block = 34;

// ---------------------------------------------------------------- activation fragments
// Activations enter the integer tensor cores as four signed 7-bit "limbs".  Per (activation row,
// super-block) a power of two 2^e >= 2 max|x| is chosen, X = rint(x * 2^(27-e)) (|X| <= 2^27) is
// split into balanced base-128 digits X = a0*2^21 + a1*2^14 + a2*2^7 + a3 with |a_j| <= 64, and
// each digit is one int8 B column: column 4*(row & 1) + j of the tile that carries activation rows
// 2*tile, 2*tile + 1.  Integer dot products with the weights are exact; the limbs are recombined
// in f32 after the per-block scales d * 2^(e-6) have been applied:
//     y = acc_0 + acc_1 * 2^-7 + acc_2 * 2^-14 + acc_3 * 2^-21.
// 28 bits cover the f32 mantissa of the block's largest elements exactly.
// The prep kernel writes, per (tile, super-block, step, lane), one 8-byte fragment {b0, b1}:
// the sub-block steps, then the per-sub-block limb sums (split into two bytes: S = 128*s1 + s0)
// and finally the f32 factor 2^(e-6) for the activation row whose columns the lane accumulates.
constexpr int kLimbs = 4;
constexpr int kRowsPerTile = 2;  // activation rows per 8-column MMA tile

FERRIC_HD size_t frag_index(size_t tile, size_t nblk, size_t blk, int steps, int s, int lane)
{
    return ((tile * nblk + blk) * (size_t)steps + (size_t)s) * 32 + (size_t)lane;
}

}  // namespace ferric
