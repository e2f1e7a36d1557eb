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
// Lane naming follows the mma.sync.m16n8k16 fragment layout: lane = 4*g + t, g = 0..7, t = 0..3.
// A fragment: regs {R0,R1,R2,R3} = (row g, k 2t..2t+1), (row g+8, k 2t..2t+1),
//                                  (row g, k 2t+8..2t+9), (row g+8, k 2t+8..2t+9).
// B fragment: regs {b0,b1} = (k 2t..2t+1, col g), (k 2t+8..2t+9, col g).
// The k index is a summation index, so any permutation is legal as long as A and B agree; the
// maps below choose the permutation that makes nibble extraction one AND per two weights.
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
// Unit (2304 B): hdr[16 rows][16 B]  |  4 segments of 512 B; segment s = 2*(row>>3) + (qs_byte>>6),
// lane 4*(row&7) + ((qs_byte>>4)&3) owns 16 bytes.
constexpr int kQ4KBlock = 144;
constexpr int kQ4KUnit = 16 * kQ4KBlock;  // 2304
constexpr int kQ4KSteps = 17;             // 16 weight steps + 1 (sub-block sums, block scale)

FERRIC_HD uint32_t q4k_unit_offset(int r, int byte)
{
    if (byte < 16) return (uint32_t)(r * 16 + byte);
    int beta = byte - 16;
    int g = r & 7, hi = r >> 3, X = beta >> 6, t = (beta >> 4) & 3;
    return (uint32_t)(256 + 512 * (2 * hi + X) + 16 * (4 * g + t) + (beta & 15));
}

// Weight index (0..255 inside the super-block) multiplied by k-slot pair j of lane t at weight
// step s = 8*X + 2*i + n:  j = 0,1 -> B reg b0 (k 2t, 2t+1);  j = 2,3 -> B reg b1 (k 2t+8, 2t+9).
FERRIC_HD int q4k_frag_weight(int s, int t, int j)
{
    int X = s >> 3, i = (s >> 1) & 3, n = s & 1;
    int byte_in_word = (j & 1) * 2 + (j >> 1);  // slots hold bytes (0,2) then (1,3) of the word
    int beta = 64 * X + 16 * t + 4 * i + byte_in_word;
    return 64 * (beta >> 5) + 32 * n + (beta & 31);
}
// Sub-block (0..7) whose 6-bit scale applies to lane t's weights at chunk X, nibble n.
FERRIC_HD int q4k_frag_subblock(int X, int t, int n) { return 2 * (2 * X + (t >> 1)) + n; }

// ---------------------------------------------------------------- Q6_K (ggml type 14)
// Raw block (crates/ferric-gguf/src/lib.rs:721-746): [ql 128][qh 64][i8 scales 16][f16 d] = 210 B.
// Unit (3360 B):
//   [   0,   32)  dpair[8]   u32: d(row g) | d(row g+8) << 16
//   [  32,  288)  sc[2][32]  u32: half hi8 = row>>3, lane 4g+t -> the 4 int8 scales of sub-blocks
//                              sb(t,k) = 8*(t>>1) + 2*k + (t&1), k = 0..3 (byte k)
//   [ 288, 2336)  ql: 4 segments of 512 B, segment 2*hi8 + c, lane 4g+t -> raw ql bytes
//                              [64*(t>>1) + 32*c + 16*(t&1), +16)
//   [2336, 3360)  qh: 2 segments of 512 B, segment hi8, lane 4g+t -> raw qh bytes [16*t, +16)
constexpr int kQ6KBlock = 210;
constexpr int kQ6KUnit = 16 * kQ6KBlock;  // 3360
constexpr int kQ6KSteps = 18;             // 16 weight steps + sub-block sums + block scale
constexpr int kQ6KOffSc = 32, kQ6KOffQl = 288, kQ6KOffQh = 2336;

FERRIC_HD uint32_t q6k_unit_offset(int r, int byte)
{
    int g = r & 7, hi = r >> 3;
    if (byte < 128) {
        int h = byte >> 6, c = (byte >> 5) & 1, t1 = (byte >> 4) & 1, t = 2 * h + t1;
        return (uint32_t)(kQ6KOffQl + 512 * (2 * hi + c) + 16 * (4 * g + t) + (byte & 15));
    }
    if (byte < 192) {
        int q = byte - 128, t = q >> 4;
        return (uint32_t)(kQ6KOffQh + 512 * hi + 16 * (4 * g + t) + (q & 15));
    }
    if (byte < 208) {
        int sb = byte - 192, h = sb >> 3, k = (sb >> 1) & 3, t1 = sb & 1, t = 2 * h + t1;
        return (uint32_t)(kQ6KOffSc + 128 * hi + 4 * (4 * g + t) + k);
    }
    return (uint32_t)(4 * g + 2 * hi + (byte - 208));
}

// Weight step s = 4*wi + k (wi = word 0..3 of the lane's 16 bytes, k = 0..3 the 32-weight group).
FERRIC_HD int q6k_frag_weight(int s, int t, int j)
{
    int wi = s >> 2, k = s & 3;
    int byte_in_word = (j & 1) * 2 + (j >> 1);
    return 128 * (t >> 1) + 32 * k + 16 * (t & 1) + 4 * wi + byte_in_word;
}
FERRIC_HD int q6k_frag_subblock(int t, int k) { return 8 * (t >> 1) + 2 * k + (t & 1); }

// ---------------------------------------------------------------- Q8_0 (ggml type 8)
// Raw block (crates/ferric-gguf/src/lib.rs:608-615): [f16 d][i8 qs 32] = 34 B, 2-byte aligned.
// Device layout: two planes, qs[rows][cols] int8 (16-byte aligned rows) and d[rows][cols/32] f16.
constexpr int kQ8Block = 34;

// ---------------------------------------------------------------- activation fragments
// The activation-preparation kernel writes, per (batch tile of 4 rows, super-block, step, lane),
// one 8-byte B fragment {b0, b1}.  Column g of the 16x8 B tile carries batch row g>>1 of the
// tile: even g the f16 head of x * 2^-e, odd g the f16 tail (x*2^-e - head) * 2^10, where 2^e is
// a per-(batch row, super-block) power of two >= max|x| so every value fits f16 whatever the
// activation range.  The final step carries the f32 factor 2^e in its second word.
constexpr float kTailScale = 1024.0f;
constexpr float kTailUnscale = 1.0f / 1024.0f;

FERRIC_HD size_t frag_index(size_t tile, size_t nblk, size_t blk, int steps, int s, int lane)
{
    return ((tile * nblk + blk) * (size_t)steps + (size_t)s) * 32 + (size_t)lane;
}

}  // namespace ferric
