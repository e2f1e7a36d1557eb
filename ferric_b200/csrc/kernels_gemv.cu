// Decode-shape (M = 1..64) packed-quant GEMV kernels for sm_100a.
//
// Replaces Tensor::matmul_q4_k / matmul_q6_k / matmul_q8_0 and their WGSL kernels
// (crates/ferric-tensor/src/dtype.rs:1426-1473 + :2995-3051, :1172-1194 + :3423-3469,
// :1292-1313 + :3473-3529) and the fused gate/up + SwiGLU kernel (:949-959, :2372-2410).
//
// Shape of the computation (Q4_K; Q6_K is analogous):
//   y[r] = sum_blk d[r,blk] * ( sum_k (sc*q)[r,k] * x[k] )  -  dmin[r,blk] * ( sum_sb m[r,sb] * Sx[sb] )
// The inner sums are integer-valued weights (sc*q <= 945, exact in f16) times activations, and run
// on the tensor cores as m16n8k16 f16 MMAs with f32 accumulation: 16 weight rows per warp, the 8
// MMA columns carrying up to four activation rows, each split into an f16 head and a scaled f16
// tail so that the product keeps f32-level accuracy.  The f32 factors d, dmin and the per-block
// activation exponent are applied to the accumulators once per super-block.  Weights stream from
// HBM exactly once, as fully coalesced 128-bit loads of the re-packed layout (layout.h).
#include "common.cuh"
#include "kernels.h"

namespace ferric {

__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hsub2_bits(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Packed f16 constants (both halves equal).
constexpr uint32_t kH2_1024 = 0x64006400u;   // 1024
constexpr uint32_t kH2_1152 = 0x64806480u;   // 1152 = 1024 + 128
constexpr uint32_t kH2_n1024 = 0xE400E400u;  // -1024
constexpr uint32_t kH2_n64 = 0xD400D400u;    // -64
constexpr uint32_t kH2_1_16 = 0x2C002C00u;   // 1/16
constexpr uint32_t kH2_n72 = 0xD480D480u;    // -72
constexpr uint32_t kH2_16 = 0x4C004C00u;     // 16
constexpr uint32_t kH2_n18432 = 0xF480F480u; // -18432
constexpr uint32_t kH2_4 = 0x44004400u;      // 4
constexpr uint32_t kH2_n4608 = 0xEC80EC80u;  // -4608
constexpr uint32_t kH2_1_4 = 0x34003400u;    // 1/4
constexpr uint32_t kH2_n288 = 0xDC80DC80u;   // -288

// ------------------------------------------------------------------------------------------
// Activation preparation: x (f32) -> B fragments (layout.h, "activation fragments").
// One warp per (batch tile of 4 rows, super-block).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t split_f16(float v, bool tail)
{
    __half h = __float2half_rn(v);
    if (tail) h = __float2half_rn((v - __half2float(h)) * kTailScale);
    return (uint32_t)__half_as_ushort(h);
}

template <int TY>
__global__ void __launch_bounds__(128) prep_kernel(const float* __restrict__ x, size_t m, size_t ldx, size_t nblk,
                                                   size_t ntiles, uint2* __restrict__ frag)
{
    constexpr int STEPS = TY == (int)kGgmlQ4K ? kQ4KSteps : kQ6KSteps;
    const size_t wid = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    if (wid >= ntiles * nblk) return;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, q = lane & 7;
    const size_t tile = wid / nblk, blk = wid % nblk;
    const size_t batch = tile * 4 + (size_t)(g >> 1);
    const bool valid = batch < m, tail = (g & 1) != 0;
    const float* xb = x + (valid ? batch : 0) * ldx + blk * 256;

    // pass 1: the 8 lanes that share a batch row scan 32 activations each
    float amax = 0.0f, s0 = 0.0f, s1 = 0.0f;
    if (valid) {
        const float4* p = reinterpret_cast<const float4*>(xb + 32 * q);
#pragma unroll
        for (int v = 0; v < 8; v++) {
            float4 f = __ldg(p + v);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
            float s = (f.x + f.y) + (f.z + f.w);
            if (v < 4) s0 += s; else s1 += s;
        }
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    int e = 0;
    if (amax > 0.0f && amax < INFINITY) {
        (void)frexpf(amax, &e);  // amax = f * 2^e with f in [0.5, 1)
        if (e < -100) e = -100;
    }
    const float down = ldexpf(1.0f, -e), up = ldexpf(1.0f, e);
    s0 *= down;
    s1 *= down;
    const int grp = lane & ~7;
    const float up_t = __shfl_sync(0xffffffffu, up, 8 * t);  // the batch row this lane's accumulators hold

    // pass 2: 16 weight steps
#pragma unroll
    for (int s = 0; s < 16; s++) {
        const int base = TY == (int)kGgmlQ4K ? q4k_frag_weight(s, t, 0) : q6k_frag_weight(s, t, 0);
        float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
        if (valid) f = __ldg(reinterpret_cast<const float4*>(xb + base));
        uint2 o;
        o.x = split_f16(f.x * down, tail) | (split_f16(f.z * down, tail) << 16);
        o.y = split_f16(f.y * down, tail) | (split_f16(f.w * down, tail) << 16);
        frag[frag_index(tile, nblk, blk, STEPS, s, lane)] = o;
    }
    if (TY == (int)kGgmlQ4K) {
        // sums over the 32-weight sub-blocks 2t, 2t+1 (lane q of the group holds sub-block q)
        const float s32 = s0 + s1;
        float a = __shfl_sync(0xffffffffu, s32, grp + 2 * t);
        float b = __shfl_sync(0xffffffffu, s32, grp + 2 * t + 1);
        uint2 o;
        o.x = split_f16(a, tail) | (split_f16(b, tail) << 16);
        o.y = __float_as_uint(up_t);
        frag[frag_index(tile, nblk, blk, STEPS, 16, lane)] = o;
    } else {
        // sums over the 16-weight sub-blocks sb(t,k): lane q holds sub-blocks 2q (s0) and 2q+1 (s1)
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int src = grp + 4 * (t >> 1) + k;
            float a = __shfl_sync(0xffffffffu, s0, src), b = __shfl_sync(0xffffffffu, s1, src);
            v[k] = (t & 1) ? b : a;
        }
        uint2 o;
        o.x = split_f16(v[0], tail) | (split_f16(v[1], tail) << 16);
        o.y = split_f16(v[2], tail) | (split_f16(v[3], tail) << 16);
        frag[frag_index(tile, nblk, blk, STEPS, 16, lane)] = o;
        frag[frag_index(tile, nblk, blk, STEPS, 17, lane)] = make_uint2(__float_as_uint(up_t), 0u);
    }
}

static int tiles_per_pass(size_t m)
{
    size_t ntiles = (m + 3) / 4;
    return ntiles >= 3 ? 4 : ntiles == 2 ? 2 : 1;
}
static size_t padded_tiles(size_t m)
{
    size_t nt = (size_t)tiles_per_pass(m), ntiles = (m + 3) / 4;
    return (ntiles + nt - 1) / nt * nt;
}

size_t frag_bytes(uint32_t ty, const DeviceWeights& w, size_t m)
{
    if (ty == kGgmlQ8_0 || m == 0) return 0;
    size_t steps = ty == kGgmlQ4K ? kQ4KSteps : kQ6KSteps;
    return padded_tiles(m) * w.nblk * steps * 32 * sizeof(uint2);
}

int32_t launch_prep(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const float* x, size_t m, size_t ldx,
                    void* frag)
{
    size_t ntiles = padded_tiles(m), warps = ntiles * w.nblk;
    if (warps == 0) return kOk;
    unsigned grid = (unsigned)((warps + 3) / 4);
    if (ty == kGgmlQ4K)
        prep_kernel<(int)kGgmlQ4K><<<grid, 128, 0, st>>>(x, m, ldx, w.nblk, ntiles, reinterpret_cast<uint2*>(frag));
    else
        prep_kernel<(int)kGgmlQ6K><<<grid, 128, 0, st>>>(x, m, ldx, w.nblk, ntiles, reinterpret_cast<uint2*>(frag));
    FERRIC_CUDA_TRY(cudaGetLastError());
    return kOk;
}

// ------------------------------------------------------------------------------------------
// Weight streaming: every warp owns a ring of kStages unit-sized slots in shared memory and keeps
// kStages-1 units in flight with 16-byte asynchronous copies (L1 bypassed), so the bytes in
// flight per SM (16 warps x 3 units x 2.3..3.4 KB) cover the HBM latency-bandwidth product
// without holding the prefetched data in registers.
// ------------------------------------------------------------------------------------------
constexpr int kStagesQ4K = 4, kStagesQ6K = 3;
constexpr int kSmemQ4K = 8 * kStagesQ4K * kQ4KUnit, kSmemQ6K = 8 * kStagesQ6K * kQ6KUnit;
extern __shared__ __align__(16) uint8_t gemv_smem[];

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src)
{
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ------------------------------------------------------------------------------------------
// Shared tail: reduce the K-split partials of a CTA in a fixed order and store.
// acc[nt][0..1] = row g (head column, tail column), acc[nt][2..3] = row g+8.
// ------------------------------------------------------------------------------------------
template <int NT, int EPI>
__device__ __forceinline__ void reduce_and_store(float (&acc)[NT][4], float (*red)[NT * 4][32], float* __restrict__ y,
                                                 size_t ldy, int rows, int m, int tile0, int wk, int rt_or_pair,
                                                 bool active)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int kpart = warp % wk, wr = warp / wk;
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) red[warp][nt * 4 + i][lane] = acc[nt][i];
    __syncthreads();
    if (kpart != 0 || !active) return;
    if (EPI == kEpiSwiglu && (wr & 1)) return;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        float v[4], u[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float s = 0.0f;
            for (int k = 0; k < wk; k++) s += red[warp + k][nt * 4 + i][lane];
            v[i] = s;
            if (EPI == kEpiSwiglu) {
                float s2 = 0.0f;
                for (int k = 0; k < wk; k++) s2 += red[warp + wk + k][nt * 4 + i][lane];
                u[i] = s2;
            }
        }
        const int batch = (tile0 + nt) * 4 + t;
        if (batch >= m) continue;
        float lo = v[0] + v[1] * kTailUnscale, hi = v[2] + v[3] * kTailUnscale;
        const int r0 = rt_or_pair * 16 + g;
        if (EPI == kEpiSwiglu) {
            float ulo = u[0] + u[1] * kTailUnscale, uhi = u[2] + u[3] * kTailUnscale;
            lo = silu_mul(lo, ulo);
            hi = silu_mul(hi, uhi);
        }
        if (r0 < rows) y[(size_t)batch * ldy + r0] = lo;
        if (r0 + 8 < rows) y[(size_t)batch * ldy + r0 + 8] = hi;
    }
}

// Which row tile a warp works on.  Plain store: consecutive tiles.  SwiGLU: even warp-rows take
// gate tile `pair`, odd warp-rows the matching up tile `pair + ff_tiles` (gate rows are stacked
// first, crates/ferric-llama/src/qwen35.rs:431).
template <int EPI>
__device__ __forceinline__ void pick_tile(int wk, int row_tiles, int ff_tiles, int& rt, int& out_tile, bool& active)
{
    const int warp = threadIdx.x >> 5, wr = warp / wk, wr_count = 8 / wk;
    if (EPI == kEpiStore) {
        rt = blockIdx.x * wr_count + wr;
        out_tile = rt;
        active = rt < row_tiles;
    } else {
        const int pair = blockIdx.x * (wr_count / 2) + (wr >> 1);
        active = pair < ff_tiles;
        rt = pair + (wr & 1) * ff_tiles;
        out_tile = pair;
    }
}

// ------------------------------------------------------------------------------------------
// Q4_K
// ------------------------------------------------------------------------------------------
struct Q4KUnit {
    uint4 hg, hh, q[4];
};
// Stage copy: the unit is mirrored byte for byte into the warp's ring slot.  Every lane copies its
// own four 16-byte quant chunks; lanes 0..15 also copy one header row each.
__device__ __forceinline__ void q4k_issue(uint8_t* slot, const uint8_t* units, size_t unit, int lane)
{
    const uint8_t* src = units + unit * kQ4KUnit;
    if (lane < 16) cp_async_16(slot + 16 * lane, src + 16 * lane);
#pragma unroll
    for (int s = 0; s < 4; s++) cp_async_16(slot + 256 + 512 * s + 16 * lane, src + 256 + 512 * s + 16 * lane);
}
__device__ __forceinline__ void q4k_read(Q4KUnit& u, const uint8_t* slot, int lane)
{
    const uint4* p = reinterpret_cast<const uint4*>(slot);
    const int g = lane >> 2;
    u.hg = p[g];
    u.hh = p[8 + g];
#pragma unroll
    for (int s = 0; s < 4; s++) u.q[s] = p[16 + 32 * s + lane];
}

struct Q4KRow {
    uint32_t mult[2][2], nbias[2][2], mins;
    float d, dmin;
};
// 6-bit scales/mins of one row's super-block -> the f16 multipliers this lane needs
// (unpack rule: crates/ferric-gguf/src/lib.rs:795-804).
__device__ __forceinline__ void q4k_row(const uint4& h, int t, Q4KRow& r)
{
    r.d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
    r.dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
    const uint32_t sc_lo = h.y & 0x3f3f3f3fu, m_lo = h.z & 0x3f3f3f3fu;
    const uint32_t sc_hi = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
    const uint32_t m_hi = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
    const int p = t >> 1;
#pragma unroll
    for (int X = 0; X < 2; X++) {
        const uint32_t word = X ? sc_hi : sc_lo;
#pragma unroll
        for (int n = 0; n < 2; n++) {
            const uint32_t byte = (uint32_t)(2 * p + n);
            const uint32_t sc2 = bytes_to_h2(word, 0x4040u | (byte * 0x0101u));  // (sc, sc)
            if (n == 0) {
                r.mult[X][n] = sc2;                               // low nibble: (1024+q)*sc - 1024*sc
                r.nbias[X][n] = hmul2_bits(sc2, kH2_n1024);
            } else {
                r.mult[X][n] = hmul2_bits(sc2, kH2_1_16);         // high nibble: (1024+16q)*sc/16 - 64*sc
                r.nbias[X][n] = hmul2_bits(sc2, kH2_n64);
            }
        }
    }
    const uint32_t mword = (t < 2) ? m_lo : m_hi;
    const uint32_t mb = (uint32_t)(2 * (t & 1));
    r.mins = bytes_to_h2(mword, 0x4040u | mb | ((mb + 1) << 8));  // (m[2t], m[2t+1])
}

template <int NT, int EPI>
__global__ void __launch_bounds__(256, (NT <= 2) ? 2 : 1)
gemv_q4k_kernel(const uint8_t* __restrict__ units, const uint2* __restrict__ frag, float* __restrict__ y, int rows,
                int nblk, int m, size_t ldy, int row_tiles, int wk, int ff_tiles)
{
    __shared__ float red[8][NT * 4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, t = lane & 3;
    int rt, out_tile;
    bool active;
    pick_tile<EPI>(wk, row_tiles, ff_tiles, rt, out_tile, active);
    const int kpart = warp % wk, per = (nblk + wk - 1) / wk;
    const int b0 = kpart * per, b1 = min(nblk, b0 + per);
    const int tile0 = blockIdx.y * NT;

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;

    if (active && b0 < b1) {
        uint8_t* ring = gemv_smem + (size_t)warp * (kStagesQ4K * kQ4KUnit);
        const size_t unit0 = (size_t)rt * nblk;
#pragma unroll
        for (int i = 0; i < kStagesQ4K - 1; i++) {
            if (b0 + i < b1) q4k_issue(ring + i * kQ4KUnit, units, unit0 + b0 + i, lane);
            cp_async_commit();
        }
        for (int b = b0; b < b1; b++) {
            const int pre = b + kStagesQ4K - 1;
            if (pre < b1) q4k_issue(ring + ((pre - b0) % kStagesQ4K) * kQ4KUnit, units, unit0 + pre, lane);
            cp_async_commit();
            cp_async_wait<kStagesQ4K - 1>();
            __syncwarp();
            Q4KUnit cur;
            q4k_read(cur, ring + ((b - b0) % kStagesQ4K) * kQ4KUnit, lane);
            __syncwarp();  // every lane has its copy before a later stage copy may overwrite the slot
            Q4KRow rg, rh;
            q4k_row(cur.hg, t, rg);
            q4k_row(cur.hh, t, rh);
            const uint2* fb[NT];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
                fb[nt] = frag + ((size_t)(tile0 + nt) * nblk + b) * (kQ4KSteps * 32) + lane;

            float cw[NT][4], cm[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) cw[nt][i] = cm[nt][i] = 0.0f;

#pragma unroll
            for (int X = 0; X < 2; X++) {
                const uint32_t wg[4] = {cur.q[X].x, cur.q[X].y, cur.q[X].z, cur.q[X].w};
                const uint32_t wh[4] = {cur.q[2 + X].x, cur.q[2 + X].y, cur.q[2 + X].z, cur.q[2 + X].w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t a = wg[i], a8 = a >> 8, c = wh[i], c8 = c >> 8;
#pragma unroll
                    for (int n = 0; n < 2; n++) {
                        const uint32_t mask = n ? 0x00f000f0u : 0x000f000fu;
                        const uint32_t A0 = hfma2_bits((a & mask) | kH2_1024, rg.mult[X][n], rg.nbias[X][n]);
                        const uint32_t A2 = hfma2_bits((a8 & mask) | kH2_1024, rg.mult[X][n], rg.nbias[X][n]);
                        const uint32_t A1 = hfma2_bits((c & mask) | kH2_1024, rh.mult[X][n], rh.nbias[X][n]);
                        const uint32_t A3 = hfma2_bits((c8 & mask) | kH2_1024, rh.mult[X][n], rh.nbias[X][n]);
                        const int s = 8 * X + 2 * i + n;
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            const uint2 bf = __ldg(fb[nt] + s * 32);
                            mma_16816(cw[nt], A0, A1, A2, A3, bf.x, bf.y);
                        }
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint2 bf = __ldg(fb[nt] + 16 * 32);
                mma_16816(cm[nt], rg.mins, rh.mins, 0u, 0u, bf.x, 0u);
                const float up = __uint_as_float(bf.y);
                const float fg = rg.d * up, fmg = -rg.dmin * up, fh = rh.d * up, fmh = -rh.dmin * up;
                acc[nt][0] = fmaf(fmg, cm[nt][0], fmaf(fg, cw[nt][0], acc[nt][0]));
                acc[nt][1] = fmaf(fmg, cm[nt][1], fmaf(fg, cw[nt][1], acc[nt][1]));
                acc[nt][2] = fmaf(fmh, cm[nt][2], fmaf(fh, cw[nt][2], acc[nt][2]));
                acc[nt][3] = fmaf(fmh, cm[nt][3], fmaf(fh, cw[nt][3], acc[nt][3]));
            }
        }
    }
    reduce_and_store<NT, EPI>(acc, red, y, ldy, EPI == kEpiSwiglu ? rows / 2 : rows, m, tile0, wk, out_tile, active);
}

// ------------------------------------------------------------------------------------------
// Q6_K
// ------------------------------------------------------------------------------------------
struct Q6KUnit {
    uint32_t dpair, scg, sch;
    uint4 ql[4], qh[2];
};
// Stage copy of one 3360-byte unit: lanes copy their own six quant chunks; lanes 0..17 also copy
// the 288 bytes of d pairs and scales.
__device__ __forceinline__ void q6k_issue(uint8_t* slot, const uint8_t* units, size_t unit, int lane)
{
    const uint8_t* src = units + unit * kQ6KUnit;
    if (lane < 18) cp_async_16(slot + 16 * lane, src + 16 * lane);
#pragma unroll
    for (int s = 0; s < 4; s++)
        cp_async_16(slot + kQ6KOffQl + 512 * s + 16 * lane, src + kQ6KOffQl + 512 * s + 16 * lane);
#pragma unroll
    for (int s = 0; s < 2; s++)
        cp_async_16(slot + kQ6KOffQh + 512 * s + 16 * lane, src + kQ6KOffQh + 512 * s + 16 * lane);
}
__device__ __forceinline__ void q6k_read(Q6KUnit& u, const uint8_t* p, int lane)
{
    u.dpair = *reinterpret_cast<const uint32_t*>(p + 4 * (lane >> 2));
    u.scg = *reinterpret_cast<const uint32_t*>(p + kQ6KOffSc + 4 * lane);
    u.sch = *reinterpret_cast<const uint32_t*>(p + kQ6KOffSc + 128 + 4 * lane);
#pragma unroll
    for (int s = 0; s < 4; s++) u.ql[s] = *reinterpret_cast<const uint4*>(p + kQ6KOffQl + 512 * s + 16 * lane);
#pragma unroll
    for (int s = 0; s < 2; s++) u.qh[s] = *reinterpret_cast<const uint4*>(p + kQ6KOffQh + 512 * s + 16 * lane);
}

struct Q6KRow {
    uint32_t lo[4], hi[4], s01, s23;
};
// The lane's four int8 sub-block scales -> f16 multipliers.  Low-nibble weights arrive as
// q*2^-24 (k = 0,1) or 16q*2^-24 (k = 2,3); high-bit pairs as h*4^k*2^-24, and must end up as
// 16*h*sc*2^-24 to line up with the low part.  All products are exact in f16.
__device__ __forceinline__ void q6k_row(uint32_t scw, Q6KRow& r)
{
    const uint32_t u = scw ^ 0x80808080u;  // bytes = sc + 128
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t v = __byte_perm(u, 0x64646464u, 0x4040u | ((uint32_t)k * 0x0101u));  // 1152 + sc, twice
        const uint32_t sc2 = hsub2_bits(v, kH2_1152);
        r.lo[k] = (k < 2) ? sc2 : hfma2_bits(v, kH2_1_16, kH2_n72);
        r.hi[k] = k == 0 ? hfma2_bits(v, kH2_16, kH2_n18432)
                : k == 1 ? hfma2_bits(v, kH2_4, kH2_n4608)
                : k == 2 ? sc2 : hfma2_bits(v, kH2_1_4, kH2_n288);
    }
    r.s01 = hsub2_bits(__byte_perm(u, 0x64646464u, 0x4140u), kH2_1152);
    r.s23 = hsub2_bits(__byte_perm(u, 0x64646464u, 0x4342u), kH2_1152);
}

template <int NT, int EPI>
__global__ void __launch_bounds__(256, (NT <= 2) ? 2 : 1)
gemv_q6k_kernel(const uint8_t* __restrict__ units, const uint2* __restrict__ frag, float* __restrict__ y, int rows,
                int nblk, int m, size_t ldy, int row_tiles, int wk, int ff_tiles)
{
    __shared__ float red[8][NT * 4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int rt, out_tile;
    bool active;
    pick_tile<EPI>(wk, row_tiles, ff_tiles, rt, out_tile, active);
    const int kpart = warp % wk, per = (nblk + wk - 1) / wk;
    const int b0 = kpart * per, b1 = min(nblk, b0 + per);
    const int tile0 = blockIdx.y * NT;

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;

    if (active && b0 < b1) {
        uint8_t* ring = gemv_smem + (size_t)warp * (kStagesQ6K * kQ6KUnit);
        const size_t unit0 = (size_t)rt * nblk;
#pragma unroll
        for (int i = 0; i < kStagesQ6K - 1; i++) {
            if (b0 + i < b1) q6k_issue(ring + i * kQ6KUnit, units, unit0 + b0 + i, lane);
            cp_async_commit();
        }
        for (int b = b0; b < b1; b++) {
            const int pre = b + kStagesQ6K - 1;
            if (pre < b1) q6k_issue(ring + ((pre - b0) % kStagesQ6K) * kQ6KUnit, units, unit0 + pre, lane);
            cp_async_commit();
            cp_async_wait<kStagesQ6K - 1>();
            __syncwarp();
            Q6KUnit cur;
            q6k_read(cur, ring + ((b - b0) % kStagesQ6K) * kQ6KUnit, lane);
            __syncwarp();
            Q6KRow rg, rh;
            q6k_row(cur.scg, rg);
            q6k_row(cur.sch, rh);
            const uint2* fb[NT];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
                fb[nt] = frag + ((size_t)(tile0 + nt) * nblk + b) * (kQ6KSteps * 32) + lane;

            float cw[NT][4], cs[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) cw[nt][i] = cs[nt][i] = 0.0f;

            const uint32_t qhg[4] = {cur.qh[0].x, cur.qh[0].y, cur.qh[0].z, cur.qh[0].w};
            const uint32_t qhh[4] = {cur.qh[1].x, cur.qh[1].y, cur.qh[1].z, cur.qh[1].w};
#pragma unroll
            for (int wi = 0; wi < 4; wi++) {
                const uint32_t hg = qhg[wi], hg8 = hg >> 8, hh = qhh[wi], hh8 = hh >> 8;
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const uint32_t lg = c ? (wi == 0 ? cur.ql[1].x : wi == 1 ? cur.ql[1].y : wi == 2 ? cur.ql[1].z : cur.ql[1].w)
                                          : (wi == 0 ? cur.ql[0].x : wi == 1 ? cur.ql[0].y : wi == 2 ? cur.ql[0].z : cur.ql[0].w);
                    const uint32_t lh = c ? (wi == 0 ? cur.ql[3].x : wi == 1 ? cur.ql[3].y : wi == 2 ? cur.ql[3].z : cur.ql[3].w)
                                          : (wi == 0 ? cur.ql[2].x : wi == 1 ? cur.ql[2].y : wi == 2 ? cur.ql[2].z : cur.ql[2].w);
                    const uint32_t lg8 = lg >> 8, lh8 = lh >> 8;
#pragma unroll
                    for (int n = 0; n < 2; n++) {
                        const int k = c + 2 * n, s = 4 * wi + k;
                        const uint32_t m4 = n ? 0x00f000f0u : 0x000f000fu;
                        const uint32_t m2 = 0x00030003u << (2 * k);
                        // low 4 bits
                        const uint32_t L0 = hmul2_bits(lg & m4, rg.lo[k]), L2 = hmul2_bits(lg8 & m4, rg.lo[k]);
                        const uint32_t L1 = hmul2_bits(lh & m4, rh.lo[k]), L3 = hmul2_bits(lh8 & m4, rh.lo[k]);
                        // high 2 bits
                        const uint32_t H0 = hmul2_bits(hg & m2, rg.hi[k]), H2 = hmul2_bits(hg8 & m2, rg.hi[k]);
                        const uint32_t H1 = hmul2_bits(hh & m2, rh.hi[k]), H3 = hmul2_bits(hh8 & m2, rh.hi[k]);
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            const uint2 bf = __ldg(fb[nt] + s * 32);
                            mma_16816(cw[nt], L0, L1, L2, L3, bf.x, bf.y);
                            mma_16816(cw[nt], H0, H1, H2, H3, bf.x, bf.y);
                        }
                    }
                }
            }
            const float dg = __half2float(__ushort_as_half((unsigned short)(cur.dpair & 0xffffu)));
            const float dh = __half2float(__ushort_as_half((unsigned short)(cur.dpair >> 16)));
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint2 bs = __ldg(fb[nt] + 16 * 32);
                mma_16816(cs[nt], rg.s01, rh.s01, rg.s23, rh.s23, bs.x, bs.y);
                const float up = __uint_as_float(__ldg(fb[nt] + 17 * 32).x);
                const float fg = dg * up, fh = dh * up;
                const float fgw = fg * 16777216.0f, fgs = fg * -32.0f, fhw = fh * 16777216.0f, fhs = fh * -32.0f;
                acc[nt][0] = fmaf(fgs, cs[nt][0], fmaf(fgw, cw[nt][0], acc[nt][0]));
                acc[nt][1] = fmaf(fgs, cs[nt][1], fmaf(fgw, cw[nt][1], acc[nt][1]));
                acc[nt][2] = fmaf(fhs, cs[nt][2], fmaf(fhw, cw[nt][2], acc[nt][2]));
                acc[nt][3] = fmaf(fhs, cs[nt][3], fmaf(fhw, cw[nt][3], acc[nt][3]));
            }
        }
    }
    reduce_and_store<NT, EPI>(acc, red, y, ldy, EPI == kEpiSwiglu ? rows / 2 : rows, m, tile0, wk, out_tile, active);
}

// ------------------------------------------------------------------------------------------
// launch
// ------------------------------------------------------------------------------------------
static int choose_wk(const DeviceWeights& w, Epilogue epi, const GemvTuning& tune)
{
    int wk = tune.wk;
    if (wk != 1 && wk != 2 && wk != 4 && wk != 8) {
        // enough warps to keep ~24 per SM busy, but at least two super-blocks per warp
        size_t tiles = w.row_tiles();
        wk = 1;
        while (wk < 8 && tiles * (size_t)wk < (size_t)tune.sm_count * 24 && w.nblk >= (size_t)(4 * wk)) wk *= 2;
    }
    if (epi == kEpiSwiglu && wk > 4) wk = 4;
    while (wk > 1 && (size_t)wk > w.nblk) wk /= 2;
    return wk;
}

template <int NT, int EPI>
static void launch_gemv_t(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const uint2* frag, size_t m, float* y,
                          size_t ldy, int wk, unsigned passes)
{
    const int row_tiles = (int)w.row_tiles(), wr = 8 / wk;
    const int ff_tiles = (int)(w.rows / 2 / 16);
    unsigned gx = EPI == kEpiStore ? (unsigned)((row_tiles + wr - 1) / wr) : (unsigned)((ff_tiles + wr / 2 - 1) / (wr / 2));
    dim3 grid(gx, passes);
    // opt in to > 48 KB of dynamic shared memory once per kernel instantiation and device
    static thread_local int attr_dev_q4 = -1, attr_dev_q6 = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (ty == kGgmlQ4K) {
        if (attr_dev_q4 != dev) {
            cudaFuncSetAttribute(gemv_q4k_kernel<NT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemQ4K);
            attr_dev_q4 = dev;
        }
        gemv_q4k_kernel<NT, EPI><<<grid, 256, kSmemQ4K, st>>>(w.units, frag, y, (int)w.rows, (int)w.nblk, (int)m, ldy,
                                                             row_tiles, wk, ff_tiles);
    } else {
        if (attr_dev_q6 != dev) {
            cudaFuncSetAttribute(gemv_q6k_kernel<NT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemQ6K);
            attr_dev_q6 = dev;
        }
        gemv_q6k_kernel<NT, EPI><<<grid, 256, kSmemQ6K, st>>>(w.units, frag, y, (int)w.rows, (int)w.nblk, (int)m, ldy,
                                                             row_tiles, wk, ff_tiles);
    }
}

int32_t launch_gemv(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const void* frag, size_t m, float* y,
                    size_t ldy, Epilogue epi, const GemvTuning& tune)
{
    if (m == 0 || w.rows == 0) return kOk;
    const int nt = tiles_per_pass(m), wk = choose_wk(w, epi, tune);
    const unsigned passes = (unsigned)(padded_tiles(m) / (size_t)nt);
    const uint2* f = reinterpret_cast<const uint2*>(frag);
#define FERRIC_GEMV_CASE(NT_)                                                                             \
    if (epi == kEpiStore) launch_gemv_t<NT_, kEpiStore>(st, ty, w, f, m, y, ldy, wk, passes);             \
    else launch_gemv_t<NT_, kEpiSwiglu>(st, ty, w, f, m, y, ldy, wk, passes)
    if (nt == 1) { FERRIC_GEMV_CASE(1); }
    else if (nt == 2) { FERRIC_GEMV_CASE(2); }
    else { FERRIC_GEMV_CASE(4); }
#undef FERRIC_GEMV_CASE
    FERRIC_CUDA_TRY(cudaGetLastError());
    return kOk;
}

// ------------------------------------------------------------------------------------------
// Q8_0: one warp per output row, lanes stride 16-weight runs, warp-shuffle reduction.
// Per 32-weight block the partial is scaled once by d, the order of the reference's CPU row
// kernel (crates/ferric-tensor/src/cpu_simd.rs:57-72).
// ------------------------------------------------------------------------------------------
template <int MB>
__global__ void __launch_bounds__(256) gemv_q8_0_kernel(const int8_t* __restrict__ qs, const uint16_t* __restrict__ dpl,
                                                        const float* __restrict__ x, int m, size_t ldx,
                                                        float* __restrict__ y, size_t ldy, int rows, int cols)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 8 + warp;
    if (row >= rows) return;
    const int batch0 = blockIdx.y * MB, nchunks = cols / 16, nb = cols / 32;
    float acc[MB];
#pragma unroll
    for (int i = 0; i < MB; i++) acc[i] = 0.0f;
    const int8_t* wrow = qs + (size_t)row * cols;
    for (int c = lane; c < nchunks; c += 32) {
        const uint4 wv = ld_stream_u4(wrow + 16 * c);
        const float d = __half2float(__ushort_as_half(dpl[(size_t)row * nb + (c >> 1)]));
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        float wf[16];
#pragma unroll
        for (int k = 0; k < 4; k++)
#pragma unroll
            for (int j = 0; j < 4; j++) wf[4 * k + j] = (float)(int8_t)((ww[k] >> (8 * j)) & 0xffu);
#pragma unroll
        for (int i = 0; i < MB; i++) {
            if (batch0 + i >= m) break;
            const float4* xp = reinterpret_cast<const float4*>(x + (size_t)(batch0 + i) * ldx + 16 * c);
            float part = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float4 xv = __ldg(xp + k);
                part = fmaf(xv.x, wf[4 * k], part);
                part = fmaf(xv.y, wf[4 * k + 1], part);
                part = fmaf(xv.z, wf[4 * k + 2], part);
                part = fmaf(xv.w, wf[4 * k + 3], part);
            }
            acc[i] = fmaf(part, d, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < MB; i++) {
        float v = acc[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && batch0 + i < m) y[(size_t)(batch0 + i) * ldy + row] = v;
    }
}

int32_t launch_gemv_q8_0(cudaStream_t st, const DeviceWeights& w, const float* x, size_t m, size_t ldx, float* y,
                         size_t ldy, const GemvTuning&)
{
    if (m == 0 || w.rows == 0) return kOk;
    dim3 grid((unsigned)((w.rows + 7) / 8), (unsigned)((m + 3) / 4));
    gemv_q8_0_kernel<4><<<grid, 256, 0, st>>>(w.q8_qs, w.q8_d, x, (int)m, ldx, y, ldy, (int)w.rows, (int)w.cols);
    FERRIC_CUDA_TRY(cudaGetLastError());
    return kOk;
}

// out[r, c] = silu(gu[r, c]) * gu[r, d + c]   (crates/ferric-tensor/src/lib.rs:2603-2618)
__global__ void swiglu_kernel(const float* __restrict__ gu, size_t t, size_t d, float* __restrict__ out)
{
    size_t total = t * d;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t r = i / d, c = i % d;
        out[i] = silu_mul(gu[r * 2 * d + c], gu[r * 2 * d + d + c]);
    }
}

int32_t launch_swiglu(cudaStream_t st, const float* gu, size_t t, size_t d, float* out)
{
    size_t total = t * d;
    if (total == 0) return kOk;
    size_t g = (total + 255) / 256;
    if (g > 148 * 32) g = 148 * 32;
    swiglu_kernel<<<(unsigned)g, 256, 0, st>>>(gu, t, d, out);
    FERRIC_CUDA_TRY(cudaGetLastError());
    return kOk;
}

}  // namespace ferric
