// Decode-shape (M = 1..64) packed-quant GEMV kernels for sm_100a.
//
// Replaces Tensor::matmul_q4_k / matmul_q6_k / matmul_q8_0 and their WGSL kernels
// (crates/ferric-tensor/src/dtype.rs:1426-1473 + :2995-3051, :1172-1194 + :3423-3469,
// :1292-1313 + :3473-3529) and the fused gate/up + SwiGLU kernel (:949-959, :2372-2410).
//
// Shape of the computation (Q4_K; Q6_K is analogous):
//   y[r] = sum_blk d[r,blk] * ( sum_sb sc[r,sb] * sum_{k in sb} q[r,k] x[k] )
//                 - dmin[r,blk] * ( sum_sb m[r,sb] * sum_{k in sb} x[k] )
// The innermost sums are integer weights times activations and run on the tensor cores as int8
// MMAs (mma.sync m16n8k32 / m16n8k16, s32 accumulate): 16 weight rows per warp, the 8 MMA columns
// carrying two activation rows as four signed 7-bit limbs each (layout.h), so the integer dot
// products are exact and the result keeps f32-level accuracy.  Nibble extraction is one AND per
// four weights; the 6-bit sub-block scales are applied to the s32 sub-block sums, and the f32
// factors d, dmin and the activation exponent once per super-block.  Weights stream from HBM
// exactly once, as fully coalesced 16-byte asynchronous copies of the re-packed layout.
#include "common.cuh"
#include "kernels.h"

namespace ferric {

// D(16x8, s32) = A(16x32, u8, row) * B(32x8, s8, col) + C
__device__ __forceinline__ void imma_16832_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1, const int (&c)[4])
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
// D(16x8, s32) = A(16x16, u8) * B(16x8, s8) + C
__device__ __forceinline__ void imma_16816_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, const int (&c)[4])
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
// D(16x8, s32) = A(16x16, s8) * B(16x8, s8) + C
__device__ __forceinline__ void imma_16816_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, const int (&c)[4])
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

// ------------------------------------------------------------------------------------------
// Activation preparation: x (f32) -> int8 limb fragments (layout.h, "activation fragments").
// One warp per (tile of 2 activation rows, super-block); 4 warps per CTA.
// ------------------------------------------------------------------------------------------
constexpr int kPrepWarps = 4;
constexpr int kNormPrepMaxWarps = 32;
constexpr int kNormPrepPushWarps = 16;   // the pushed-exchange variant holds every rank's values in registers while it polls
constexpr int kNormPrepWideWarps = 8;    // ... and with more than two ranks it needs still more registers per thread

// Per-warp staging.  16-byte aligned (and so padded to a multiple of 16 bytes): the limb rows are
// written with 128-bit stores, and the struct is used in arrays indexed by warp.
struct __align__(16) PrepSmem {
    int8_t limb[2][kLimbs][256];  // limb bytes [row 0..1][limb 0..3][256]
    int sum[2][kLimbs][16];       // 16-weight limb sums
    float up[2];                  // 2^(e-6) per row
};
static_assert(sizeof(PrepSmem) % 16 == 0, "PrepSmem must keep 16-byte alignment inside arrays");

// One warp turns 2 x 256 activations (lanes 0..15: row 0, lanes 16..31: row 1; 16 values each, in
// v[]) into the fragments of (tile, blk).
template <int TY>
__device__ __forceinline__ void prep_block(const float (&v)[16], PrepSmem& sm, size_t tile, size_t nblk, size_t blk,
                                           uint2* __restrict__ frag)
{
    const int lane = threadIdx.x & 31, prow = lane >> 4, q = lane & 15;
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    int e = 0;
    if (amax > 0.0f && amax < INFINITY) {
        (void)frexpf(amax, &e);  // amax = f * 2^e, f in [0.5, 1)
        e += 1;                  // 2^e >= 2 max|x|, so |x| 2^-e <= 1/2
        if (e < -80) e = -80;
        if (e > 120) e = 120;
    }
    const float to_int = ldexpf(1.0f, 27 - e);  // X = rint(x * 2^(27-e)), |X| <= 2^27
    int sum[kLimbs] = {0, 0, 0, 0};
    uint32_t packed[kLimbs][4];
#pragma unroll
    for (int i = 0; i < 16; i++) {
        int X = __float2int_rn(v[i] * to_int);
        int a3 = ((X + 64) & 127) - 64; X = (X - a3) >> 7;
        int a2 = ((X + 64) & 127) - 64; X = (X - a2) >> 7;
        int a1 = ((X + 64) & 127) - 64; X = (X - a1) >> 7;
        int a0 = X;
        const int w = i >> 2, sh = 8 * (i & 3);
        if ((i & 3) == 0) packed[0][w] = packed[1][w] = packed[2][w] = packed[3][w] = 0u;
        packed[0][w] |= (uint32_t)(a0 & 0xff) << sh;
        packed[1][w] |= (uint32_t)(a1 & 0xff) << sh;
        packed[2][w] |= (uint32_t)(a2 & 0xff) << sh;
        packed[3][w] |= (uint32_t)(a3 & 0xff) << sh;
        sum[0] += a0; sum[1] += a1; sum[2] += a2; sum[3] += a3;
    }
#pragma unroll
    for (int j = 0; j < kLimbs; j++) {
        *reinterpret_cast<uint4*>(&sm.limb[prow][j][16 * q]) = make_uint4(packed[j][0], packed[j][1], packed[j][2], packed[j][3]);
        sm.sum[prow][j][q] = sum[j];
    }
    if (q == 0) sm.up[prow] = ldexpf(1.0f, e - 6);
    __syncwarp();

    // fragments.  B layout: lane = 4*g + t, column g = 4*(row in tile) + limb.
    const int g = lane >> 2, t = lane & 3, brow = g >> 2, limb = g & 3;
    const int8_t* lb = sm.limb[brow][limb];
    const int* ss = sm.sum[brow][limb];
    constexpr int STEPS = TY == (int)kGgmlQ4K ? kQ4KSteps : kQ6KSteps;
    uint2* out = frag + frag_index(tile, nblk, blk, STEPS, 0, lane);
#pragma unroll
    for (int s = 0; s < 8; s++) {
        uint2 o;
        if (TY == (int)kGgmlQ4K) {  // sub-block s: weights 32s + 8t + 0..7
            o = *reinterpret_cast<const uint2*>(lb + 32 * s + 8 * t);
        } else {                    // sub-blocks 2s, 2s+1: weights 16sb + 4t + 0..3
            o.x = *reinterpret_cast<const uint32_t*>(lb + 32 * s + 4 * t);
            o.y = *reinterpret_cast<const uint32_t*>(lb + 32 * s + 16 + 4 * t);
        }
        out[s * 32] = o;
    }
    // limb sums per sub-block, S = 128*s1 + s0 with |s0| <= 64: k slot 4t + i <-> sub-block 4t + i
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int S;
        if (TY == (int)kGgmlQ4K) {
            const int sb = 4 * t + i;  // 8 sub-blocks of 32 weights; k slots 8..15 stay zero
            S = sb < 8 ? ss[2 * sb] + ss[2 * sb + 1] : 0;
        } else {
            S = ss[4 * t + i];
        }
        const int s0 = ((S + 64) & 127) - 64, s1 = (S - s0) >> 7;
        lo |= (uint32_t)(s0 & 0xff) << (8 * i);
        hi |= (uint32_t)(s1 & 0xff) << (8 * i);
    }
    out[8 * 32] = make_uint2(lo, hi);
    // the C layout gives this lane columns 2t, 2t+1 = activation row t>>1 of the tile
    out[9 * 32] = make_uint2(__float_as_uint(sm.up[t >> 1]), 0u);
    __syncwarp();
}

template <int TY>
__global__ void __launch_bounds__(32 * kPrepWarps)
prep_kernel(const float* __restrict__ x, size_t m, size_t ldx, size_t nblk, size_t ntiles, uint2* __restrict__ frag)
{
    __shared__ __align__(16) PrepSmem sm[kPrepWarps];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t wid = blockIdx.x * (size_t)kPrepWarps + warp;
    if (wid >= ntiles * nblk) return;
    const size_t tile = wid / nblk, blk = wid % nblk;
    const size_t batch = tile * kRowsPerTile + (size_t)(lane >> 4);
    float v[16];
    if (batch < m) {
        const float4* p = reinterpret_cast<const float4*>(x + batch * ldx + blk * 256 + 16 * (lane & 15));
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float4 f = ld_act(p + i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = 0.0f;
    }
    prep_block<TY>(v, sm[warp], tile, nblk, blk, frag);
}

// Every wait on a peer is bounded (PeerSum / PushSrc::wait_spins, about a second of polling by default): when it runs
// out the kernel records the failure in the exchange's status word and carries on.

// Sum of all ranks' partials at float offset `off`, in rank order (the same order on every rank,
// so every rank forms bit-identical sums).  Peer memory is read uncached: it changes between
// exchanges while this SM may still hold lines of the previous one.
__device__ __forceinline__ float4 peer_sum4(const PeerSum& p, size_t off)
{
    // All loads are issued before the first sum, so the peers' latencies overlap instead of adding up; the sum
    // itself runs in rank order.  Fully unrolled so that the pointer table stays in the kernel's parameter space.
    float4 v[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; r++) {
        v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < p.world)
            asm volatile("ld.global.cv.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v[r].x), "=f"(v[r].y), "=f"(v[r].z), "=f"(v[r].w) : "l"(p.part[r] + off));
    }
    float4 s = v[0];
#pragma unroll
    for (int r = 1; r < kMaxRanks; r++) {
        if (r < p.world) {
            s.x += v[r].x; s.y += v[r].y; s.z += v[r].z; s.w += v[r].w;
        }
    }
    return s;
}

// Pushed exchange, consumer side: R runs of four values starting at pair offset `off` of every rank's slice, each value
// polled (bounded) until its stamp is `want`, summed in rank order.  All loads of a round are issued before the first
// check, so a round costs one trip to L2 however many ranks and runs it covers; WMAX (the largest world size this
// instantiation serves) and R are traded against each other to keep the values in flight in registers.
template <int R, int WMAX>
__device__ __forceinline__ void pushed_sum(const PushSrc& p, const uint2* base, size_t off, unsigned want, int limit, float4* out)
{
    uint4 a[WMAX][R], b[WMAX][R];
    int spins = 0;
    for (;;) {
#pragma unroll
        for (int r = 0; r < WMAX; r++) {
            if (r < p.world) {
#pragma unroll
                for (int j = 0; j < R; j++) {
                    const uint2* src = base + (size_t)r * p.elems + off + 4 * j;
                    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a[r][j].x), "=r"(a[r][j].y), "=r"(a[r][j].z), "=r"(a[r][j].w) : "l"(src));
                    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b[r][j].x), "=r"(b[r][j].y), "=r"(b[r][j].z), "=r"(b[r][j].w) : "l"(src + 2));
                }
            }
        }
        bool ok = true;
#pragma unroll
        for (int r = 0; r < WMAX; r++)
            if (r < p.world)
#pragma unroll
                for (int j = 0; j < R; j++) ok = ok && a[r][j].y == want && a[r][j].w == want && b[r][j].y == want && b[r][j].w == want;
        if (ok) break;
        if (++spins > limit) {
            *p.status = 1;
            break;
        }
    }
#pragma unroll
    for (int j = 0; j < R; j++) {
        float4 s = make_float4(__uint_as_float(a[0][j].x), __uint_as_float(a[0][j].z), __uint_as_float(b[0][j].x), __uint_as_float(b[0][j].z));
#pragma unroll
        for (int r = 1; r < WMAX; r++) {
            if (r < p.world) {
                s.x += __uint_as_float(a[r][j].x); s.y += __uint_as_float(a[r][j].z);
                s.z += __uint_as_float(b[r][j].x); s.w += __uint_as_float(b[r][j].z);
            }
        }
        out[j] = s;
    }
}

// Publish this rank's next exchange count to every peer (one thread per peer).
__global__ void tp_signal_kernel(unsigned* epoch, unsigned* const* peer_flag_slots, int world)
{
    __shared__ unsigned e;
    pdl_launch_dependents();
    pdl_wait();  // the product whose result is being announced is complete and visible
    if (threadIdx.x == 0) {
        e = *epoch + 1;
        *epoch = e;
    }
    __syncthreads();
    if ((int)threadIdx.x < world) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flag_slots[threadIdx.x]), "r"(e) : "memory");
    }
}

int32_t launch_tp_signal(cudaStream_t st, unsigned* epoch, unsigned* const* peer_flag_slots, int world,
                         const GemvTuning& tune)
{
    FERRIC_CUDA_TRY(launch_kernel(tp_signal_kernel, dim3(1), dim3(32), 0, st, tune.pdl, epoch, peer_flag_slots, world));
    return kOk;
}

// Fused residual add + RMSNorm + activation preparation (crates/ferric-tensor/src/lib.rs:372-384
// followed by the matmul's own input conversion).  One CTA per tile of 2 activation rows; warp w
// handles super-blocks w, w + nwarps, ...
// Thread-block cluster helpers of the pushed consumer (a launch without clusters reads rank 0 of 1).
__device__ __forceinline__ unsigned cl_rank()
{
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned cl_size()
{
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cl_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float cl_load_f32(const float* own_smem, unsigned rank)
{
    unsigned a;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"((unsigned)__cvta_generic_to_shared(own_smem)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}

// PEERS: 0 no exchange, 1 partial sums pulled from the peers' memory after their signal, 2 partial sums the peers
// pushed into this rank's memory.
// WMAX (pushed form only): the largest world size the instantiation serves; up to 2 ranks CTAs of up to 16 warps
// polls all 16 of a lane's values in one round, above that CTAs of up to 8 warps (the tile is spread over a cluster)
// poll 8 values per round.
template <int TY, int PEERS, int WMAX>
__global__ void __launch_bounds__(PEERS == 2 ? (WMAX <= 2 ? 32 * kNormPrepPushWarps : 32 * kNormPrepWideWarps) : PEERS == 0 ? 32 * kNormPrepPushWarps : 32 * kNormPrepMaxWarps)
norm_prep_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ wgt, float eps,
                 size_t m, size_t d, size_t nblk, float* __restrict__ sum, float* __restrict__ norm,
                 uint2* __restrict__ frag, PeerSum peers, PushSrc pushed)
{
    extern __shared__ __align__(16) uint8_t np_smem[];
    PrepSmem* sm = reinterpret_cast<PrepSmem*>(np_smem);
    __shared__ float part[2][kNormPrepMaxWarps];
    pdl_launch_dependents();
    pdl_wait();
    unsigned want = 0;
    const uint2* recv = nullptr;
    int wait_limit = 0;
    if (PEERS == 2) {
        // a wait that ran out earlier stays recorded: later kernels then do not wait again, so a lost peer costs one
        // bound, not one per kernel
        wait_limit = *reinterpret_cast<volatile int*>(pushed.status) ? 0 : pushed.wait_spins;
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(want) : "l"(pushed.epoch));
        want += 1;
        recv = pushed.recv + (size_t)(want & 1) * pushed.world * pushed.elems;
    }
    if (PEERS == 1) {
        // every rank's partial must have arrived: peers publish their exchange count into this
        // rank's flag slots; wait (bounded) until each has reached this rank's own count
        if (threadIdx.x < peers.world && *reinterpret_cast<volatile int*>(peers.status) == 0) {
            const unsigned want = *peers.epoch;
            unsigned seen = 0;
            int spins = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(peers.flags + threadIdx.x) : "memory");
                if ((int)(seen - want) >= 0) break;
                if (++spins > peers.wait_spins) {
                    *peers.status = 1;
                    break;
                }
            }
        }
        __syncthreads();
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int prow = lane >> 4, q = lane & 15;
    // The pushed form may run one tile on a cluster of CTAs: polling every rank's pairs is a lot of L2 traffic for
    // one SM, so the super-blocks are dealt round the cluster and only the sums of squares cross it.
    const unsigned crank = PEERS != 1 ? cl_rank() : 0u, csize = PEERS != 1 ? cl_size() : 1u;
    const size_t blk_first = (size_t)crank * nwarps + warp, blk_step = (size_t)csize * nwarps;
    const size_t tile = blockIdx.x / csize, batch = tile * kRowsPerTile + (size_t)prow;
    const bool valid = batch < m;
    // pass 1: s = a + b, sum of squares per row.  A warp's first block stays in registers for pass 2 (with enough warps
    // that is its only block), which saves the second trip to memory.
    constexpr bool kKeep = PEERS != 1;
    float4 keep[4];
    float ms = 0.0f;
    for (size_t blk = blk_first; blk < nblk; blk += blk_step) {
        if (valid) {
            const size_t off = batch * d + blk * 256 + 16 * q;
            float4 gp[4];
            if (PEERS == 2) {
                constexpr int R = WMAX <= 2 ? 4 : 2;
#pragma unroll
                for (int i0 = 0; i0 < 4; i0 += R) pushed_sum<R, (WMAX > 0 ? WMAX : 1)>(pushed, recv, off + 4 * i0, want, wait_limit, gp + i0);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float4 f = ld_act(reinterpret_cast<const float4*>(a + off) + i);
                if (b) {
                    const float4 g = ld_act(reinterpret_cast<const float4*>(b + off) + i);
                    f.x += g.x; f.y += g.y; f.z += g.z; f.w += g.w;
                }
                if (PEERS == 1) {
                    const float4 g = peer_sum4(peers, off + 4 * i);
                    f.x += g.x; f.y += g.y; f.z += g.z; f.w += g.w;
                }
                if (PEERS == 2) {
                    f.x += gp[i].x; f.y += gp[i].y; f.z += gp[i].z; f.w += gp[i].w;
                }
                if (sum) reinterpret_cast<float4*>(sum + off)[i] = f;
                if (kKeep && blk == blk_first) keep[i] = f;
                ms = fmaf(f.x, f.x, ms); ms = fmaf(f.y, f.y, ms); ms = fmaf(f.z, f.z, ms); ms = fmaf(f.w, f.w, ms);
            }
        }
    }
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) ms += __shfl_xor_sync(0xffffffffu, ms, o);
    if (q == 0) part[prow][warp] = ms;
    __syncthreads();
    float tot = 0.0f;
    if (PEERS != 1 && csize > 1) {
        // every CTA adds all the cluster's per-warp sums in super-block order: the same order in every CTA, and the
        // order of a single CTA with one warp per super-block
        cl_sync();
        for (unsigned c = 0; c < csize; c++)
            for (int i = 0; i < nwarps; i++) tot += cl_load_f32(&part[prow][i], c);
    } else {
        for (int i = 0; i < nwarps; i++) tot += part[prow][i];
    }
    const float inv = 1.0f / sqrtf(tot / (float)d + eps);
    // pass 2: normalise and convert
    for (size_t blk = blk_first; blk < nblk; blk += blk_step) {
        float v[16];
        if (valid) {
            const size_t off = batch * d + blk * 256 + 16 * q;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float4 f;
                if (kKeep && blk == blk_first) {
                    f = keep[i];
                } else if (sum || PEERS == 2) {   // the pushed form always writes the sum (its launcher insists)
                    f = reinterpret_cast<const float4*>(sum + off)[i];
                } else {
                    f = ld_act(reinterpret_cast<const float4*>(a + off) + i);
                    if (b) {
                        const float4 g = ld_act(reinterpret_cast<const float4*>(b + off) + i);
                        f.x += g.x; f.y += g.y; f.z += g.z; f.w += g.w;
                    }
                    if (PEERS == 1) {
                        const float4 g = peer_sum4(peers, off + 4 * i);
                        f.x += g.x; f.y += g.y; f.z += g.z; f.w += g.w;
                    }
                }
                float4 w4 = make_float4(1.f, 1.f, 1.f, 1.f);
                if (wgt) w4 = __ldg(reinterpret_cast<const float4*>(wgt + blk * 256 + 16 * q) + i);
                f.x = f.x * inv * w4.x; f.y = f.y * inv * w4.y; f.z = f.z * inv * w4.z; f.w = f.w * inv * w4.w;
                if (norm) reinterpret_cast<float4*>(norm + off)[i] = f;
                v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = 0.0f;
        }
        prep_block<TY>(v, sm[warp], tile, nblk, blk, frag);
    }
    if (PEERS != 1 && csize > 1) cl_sync();   // no CTA leaves while another may still read its sums
    if (PEERS == 2) {
        // the last CTA to get here closes the exchange: the next one of this kind carries the next number
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(pushed.ticket, 1u) == gridDim.x - 1) {
                *pushed.ticket = 0;
                asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(pushed.epoch), "r"(want) : "memory");
            }
        }
    }
}

// Activation tiles (of two rows) a launch pass covers.  Two at most: a warp that carries four tiles needs over 200
// registers, which leaves one CTA per SM, and measured slower than two passes of two tiles that re-read the weights
// (gate|up at 8 rows: 56.8 us against 48.7 us; the 64-layer step 11.0 ms against 8.6 ms).
static int tiles_per_pass(size_t m)
{
    size_t ntiles = (m + kRowsPerTile - 1) / kRowsPerTile;
    return ntiles >= 2 ? 2 : 1;
}
static size_t padded_tiles(size_t m)
{
    size_t nt = (size_t)tiles_per_pass(m), ntiles = (m + kRowsPerTile - 1) / kRowsPerTile;
    return (ntiles + nt - 1) / nt * nt;
}

size_t gemv_padded_tiles(size_t m) { return padded_tiles(m); }

size_t frag_bytes(uint32_t ty, const DeviceWeights& w, size_t m)
{
    if (!has_prepared_form(ty) || m == 0) return 0;
    size_t steps = (ty == kGgmlQ4K || ty == kGgmlQ5K) ? kQ4KSteps : kQ6KSteps;   // Q5_K shares Q4_K's fragments
    return padded_tiles(m) * w.nblk * steps * 32 * sizeof(uint2);
}

int32_t launch_prep(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const float* x, size_t m, size_t ldx,
                    void* frag, const GemvTuning& tune)
{
    size_t ntiles = padded_tiles(m), warps = ntiles * w.nblk;
    if (warps == 0) return kOk;
    dim3 grid((unsigned)((warps + kPrepWarps - 1) / kPrepWarps)), block(32 * kPrepWarps);
    uint2* f = reinterpret_cast<uint2*>(frag);
    if (ty == kGgmlQ4K || ty == kGgmlQ5K)
        FERRIC_CUDA_TRY(launch_kernel(prep_kernel<(int)kGgmlQ4K>, grid, block, 0, st, tune.pdl, x, m, ldx, w.nblk, ntiles, f));
    else
        FERRIC_CUDA_TRY(launch_kernel(prep_kernel<(int)kGgmlQ6K>, grid, block, 0, st, tune.pdl, x, m, ldx, w.nblk, ntiles, f));
    return kOk;
}

int32_t launch_norm_prep(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const float* a, const float* b,
                         const float* weight, float eps, size_t m, float* sum, float* norm, void* frag,
                         const GemvTuning& tune, const PeerSum& peers, const PushSrc& pushed)
{
    size_t ntiles = padded_tiles(m);
    if (ntiles == 0 || w.nblk == 0) return kOk;
    const int mode = pushed.world > 2 ? 3 : pushed.world > 0 ? 2 : peers.world > 0 ? 1 : 0;
    const int max_warps = mode == 3 ? kNormPrepWideWarps : (mode == 2 || mode == 0) ? kNormPrepPushWarps : kNormPrepMaxWarps;
    unsigned cluster = 1;
    if (mode == 0 && w.nblk >= 8) cluster = 4;   // one CTA alone is latency-bound on a 5120-wide row (8 us); four share the blocks
    if (mode >= 2) {
        int c = tune.push_cluster > 0 ? tune.push_cluster : (pushed.world > 2 ? 4 : w.nblk > (size_t)kNormPrepPushWarps ? 2 : 1);
        while (c > 1 && ((c & (c - 1)) || c > 8 || (size_t)c > w.nblk)) c--;   // a power of two up to 8, at most one CTA per super-block
        cluster = (unsigned)c;
    }
    const size_t per_cta = (w.nblk + cluster - 1) / cluster;
    int nwarps = (int)(per_cta < (size_t)max_warps ? per_cta : (size_t)max_warps);
    dim3 grid((unsigned)ntiles * cluster), block(32 * nwarps);
    size_t smem = (size_t)nwarps * sizeof(PrepSmem);
    uint2* f = reinterpret_cast<uint2*>(frag);
    using Kernel = void (*)(const float*, const float*, const float*, float, size_t, size_t, size_t, float*, float*, uint2*,
                            PeerSum, PushSrc);
    // the variant without an exchange carries none of the peer-pointer code
    static const Kernel table[2][4] = {
        {norm_prep_kernel<(int)kGgmlQ4K, 0, 0>, norm_prep_kernel<(int)kGgmlQ4K, 1, 0>, norm_prep_kernel<(int)kGgmlQ4K, 2, 2>,
         norm_prep_kernel<(int)kGgmlQ4K, 2, kMaxRanks>},
        {norm_prep_kernel<(int)kGgmlQ6K, 0, 0>, norm_prep_kernel<(int)kGgmlQ6K, 1, 0>, norm_prep_kernel<(int)kGgmlQ6K, 2, 2>,
         norm_prep_kernel<(int)kGgmlQ6K, 2, kMaxRanks>}};
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    const int max_smem = (int)(kNormPrepMaxWarps * sizeof(PrepSmem));
    if (attr_dev != dev) {
        for (int i = 0; i < 2; i++)
            for (int j = 0; j < 4; j++) cudaFuncSetAttribute(table[i][j], cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
        attr_dev = dev;
    }
    Kernel kernel = table[(ty == kGgmlQ4K || ty == kGgmlQ5K) ? 0 : 1][mode];
    if (cluster > 1)
        FERRIC_CUDA_TRY(launch_kernel_cluster(kernel, grid, block, smem, st, tune.pdl, cluster, a, b, weight, eps, m, w.cols, w.nblk, sum,
                                              norm, f, peers, pushed));
    else
        FERRIC_CUDA_TRY(launch_kernel(kernel, grid, block, smem, st, tune.pdl, a, b, weight, eps, m, w.cols, w.nblk, sum, norm, f, peers, pushed));
    return kOk;
}

// ------------------------------------------------------------------------------------------
// Weight streaming: every warp owns a ring of kStages unit-sized slots in shared memory and keeps
// kStages-1 units in flight with 16-byte asynchronous copies (L1 bypassed), so the bytes in
// flight per SM cover the HBM latency-bandwidth product without holding prefetched data in
// registers.
// ------------------------------------------------------------------------------------------
constexpr int kStagesQ4K = 4, kStagesQ6K = 3;
constexpr int kSmemQ4K = 8 * kStagesQ4K * kQ4KUnit, kSmemQ5K = 8 * kStagesQ4K * kQ5KUnit, kSmemQ6K = 8 * kStagesQ6K * kQ6KUnit;
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
// Shared tail: reduce the K-split partials of a CTA in a fixed order, recombine the limbs, store.
// acc[nt][0..1] = row g, columns 2t, 2t+1 (activation row t>>1, limbs 2(t&1), 2(t&1)+1);
// acc[nt][2..3] = row g+8.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void push_pair(uint2* dst, float v, unsigned stamp)
{
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(v)), "r"(stamp) : "memory");
}

// One lane's two results (rows r0 and r0 + 8 of activation row `batch`): into y, or, for the pushed exchange, as
// (value, exchange number) pairs into every rank's receive region (8-byte stores arrive whole).
template <int EPI>
__device__ __forceinline__ void store_result(float* __restrict__ y, size_t ldy, int rows, int batch, int r0, float lo, float hi,
                                             const PushDst& push)
{
    if (EPI == kEpiPush) {
        unsigned stamp;
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(stamp) : "l"(push.epoch));
        stamp += 1;
        const size_t at = (size_t)(stamp & 1) * push.parity_stride + (size_t)batch * ldy + r0;
#pragma unroll
        for (int r = 0; r < kMaxRanks; r++) {
            if (r < push.world) {
                if (r0 < rows) push_pair(push.dst[r] + at, lo, stamp);
                if (r0 + 8 < rows) push_pair(push.dst[r] + at + 8, hi, stamp);
            }
        }
    } else {
        if (r0 < rows) y[(size_t)batch * ldy + r0] = lo;
        if (r0 + 8 < rows) y[(size_t)batch * ldy + r0 + 8] = hi;
    }
}

// The job of a chain link (kernels.h, ChainJob): turn block `blk` of the result -- complete in memory, or, for the
// pushed exchange, arriving in this rank's receive region -- into the next product's activation fragments.  Run by one
// whole warp; `sm` is scratch of that warp (its weight ring, drained by now).
template <int EPI>
__device__ __forceinline__ void chain_job(const ChainJob& j, int blk, int m, PrepSmem& sm)
{
    const int lane = threadIdx.x & 31, prow = lane >> 4, q = lane & 15;
    if (!(EPI == kEpiPush && j.kind == 3)) __threadfence();   // the other tiles' stores came before their tickets
    unsigned want = 0;
    const uint2* recv = nullptr;
    int wait_limit = 0;
    if (EPI == kEpiPush && j.kind == 3) {
        wait_limit = *reinterpret_cast<volatile int*>(j.pushed.status) ? 0 : j.pushed.wait_spins;
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(want) : "l"(j.pushed.epoch));
        want += 1;
        recv = j.pushed.recv + (size_t)(want & 1) * j.pushed.world * j.pushed.elems;
    }
    const size_t nblk = (size_t)j.blocks, d = nblk * 256;
    for (int tile = 0; tile < j.tiles; tile++) {
        const size_t batch = (size_t)tile * kRowsPerTile + (size_t)prow;
        const bool valid = batch < (size_t)m;   // the same for the 16 lanes of a row
        float4 f[4];
        float ms = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) f[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (valid) {
            if (EPI == kEpiPush && j.kind == 3) {
                // as many of the lane's 16 values per polling round as the registers hold for the group's size
                const size_t off = batch * d + (size_t)blk * 256 + 16 * q;
                if (j.pushed.world <= 2) {
                    pushed_sum<4, 2>(j.pushed, recv, off, want, wait_limit, f);
                } else {
#pragma unroll 1
                    for (int i = 0; i < 4; i++) pushed_sum<1, kMaxRanks>(j.pushed, recv, off + 4 * i, want, wait_limit, f + i);
                }
            } else {
                const float4* yp = reinterpret_cast<const float4*>(j.y + batch * j.ldy + (size_t)blk * 256 + 16 * q);
#pragma unroll
                for (int i = 0; i < 4; i++) f[i] = __ldcg(yp + i);
            }
            if (j.kind >= 2) {
                float4* hp = reinterpret_cast<float4*>(j.h + batch * d + (size_t)blk * 256 + 16 * q);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 a = __ldcg(hp + i);
                    f[i].x = a.x + f[i].x; f[i].y = a.y + f[i].y; f[i].z = a.z + f[i].z; f[i].w = a.w + f[i].w;
                    hp[i] = f[i];
                    ms = fmaf(f[i].x, f[i].x, ms); ms = fmaf(f[i].y, f[i].y, ms); ms = fmaf(f[i].z, f[i].z, ms); ms = fmaf(f[i].w, f[i].w, ms);
                }
            }
        }
        if (j.kind >= 2) {
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) ms += __shfl_xor_sync(0xffffffffu, ms, o);
            if (valid && q == 0) j.ssq[batch * nblk + (size_t)blk] = ms;
            if (valid && j.weight) {
                const float4* wp = reinterpret_cast<const float4*>(j.weight + (size_t)blk * 256 + 16 * q);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 w4 = __ldg(wp + i);
                    f[i].x *= w4.x; f[i].y *= w4.y; f[i].z *= w4.z; f[i].w *= w4.w;
                }
            }
        }
        float v[16];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[4 * i] = f[i].x; v[4 * i + 1] = f[i].y; v[4 * i + 2] = f[i].z; v[4 * i + 3] = f[i].w;
        }
        __syncwarp();
        if (j.out_ty == (int)kGgmlQ6K) prep_block<(int)kGgmlQ6K>(v, sm, (size_t)tile, nblk, (size_t)blk, j.frag);
        else prep_block<(int)kGgmlQ4K>(v, sm, (size_t)tile, nblk, (size_t)blk, j.frag);
    }
    if (lane == 0) j.tickets[blk] = 0;   // ready for the next launch
    if (EPI == kEpiPush && j.kind == 3) {
        // the last job to finish closes the exchange: every tile of this launch has been pushed by then
        __threadfence();
        __syncwarp();
        if (lane == 0 && atomicAdd(j.done, 1u) == (unsigned)j.blocks - 1u) {
            *j.done = 0;
            asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(j.pushed.epoch), "r"(want) : "memory");
        }
    }
}

// 1 / sqrt(mean of squares + eps) of the activation rows this lane's result columns belong to (Chain::ssq_in).  The
// per-block sums are fetched by the whole warp at once (one trip to L2 for all of them) and added in a fixed order --
// a lane's blocks in turn, then a butterfly over the lanes -- so every warp of every CTA forms the same bits.
template <int NT, bool CHAIN>
__device__ __forceinline__ void chain_scales(float (&inv)[NT], const Chain& chain, int tile0, int m)
{
#pragma unroll
    for (int nt = 0; nt < NT; nt++) inv[nt] = 1.0f;
    if (CHAIN && chain.ssq_in) {
        const int lane = threadIdx.x & 31, t = lane & 3;
        float tot[NT][kRowsPerTile];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int r = 0; r < kRowsPerTile; r++) {
                const int batch = (tile0 + nt) * kRowsPerTile + r;
                float s = 0.0f;
                if (batch < m)
                    for (int i = lane; i < chain.ssq_blocks; i += 32) s += __ldcg(chain.ssq_in + (size_t)batch * chain.ssq_blocks + i);
                tot[nt][r] = s;
            }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
#pragma unroll
            for (int r = 0; r < kRowsPerTile; r++)
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) tot[nt][r] += __shfl_xor_sync(0xffffffffu, tot[nt][r], o);
            const int batch = (tile0 + nt) * kRowsPerTile + (t >> 1);
            if (batch < m) inv[nt] = 1.0f / sqrtf(((t >> 1) ? tot[nt][1] : tot[nt][0]) / chain.d + chain.eps);
        }
    }
}

// Indexed product: which expert, activation row and result row this launch pass (blockIdx.y) works on.
struct IdPick {
    int batch = -1, out = 0, expert = 0;
    bool ok = true;
};
__device__ __forceinline__ IdPick id_pick(const IdSel& id)
{
    IdPick p;
    const int pair = blockIdx.y, tok = pair / id.k, slot = pair - tok * id.k;
    const float fe = __ldcg(id.selw + (size_t)tok * 2 * id.k + id.k + slot);
    p.expert = (int)fe;
    p.ok = p.expert >= 0 && p.expert < id.n_expert;
    if (!p.ok) p.expert = 0;
    p.batch = id.x_per_pair ? pair : tok;
    p.out = pair;
    return p;
}

template <int NT, int EPI, bool CHAIN = false>
__device__ __forceinline__ void reduce_and_store(float (&acc)[NT][4], float (*red)[NT * 4][32], float* __restrict__ y,
                                                 size_t ldy, int rows, int m, int tile0, int wk, int out_tile,
                                                 bool active, const PushDst& push, const float (&inv)[NT], const Chain& chain,
                                                 uint8_t* warp_smem, int id_batch = -1, int id_out = 0, bool id_ok = true)
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
    // limb weights of this lane's two columns: 2^(-7*limb)
    const float w0 = (t & 1) ? 6.103515625e-05f : 1.0f;          // 2^-14 : 2^0
    const float w1 = (t & 1) ? 4.76837158203125e-07f : 0.0078125f; // 2^-21 : 2^-7
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
        float lo = v[0] * w0 + v[1] * w1, hi = v[2] * w0 + v[3] * w1;
        lo += __shfl_xor_sync(0xffffffffu, lo, 1);
        hi += __shfl_xor_sync(0xffffffffu, hi, 1);
        if (CHAIN) {
            lo *= inv[nt];
            hi *= inv[nt];
        }
        if (EPI == kEpiSwiglu) {
            float ulo = u[0] * w0 + u[1] * w1, uhi = u[2] * w0 + u[3] * w1;
            ulo += __shfl_xor_sync(0xffffffffu, ulo, 1);
            uhi += __shfl_xor_sync(0xffffffffu, uhi, 1);
            if (CHAIN) {
                ulo *= inv[nt];
                uhi *= inv[nt];
            }
            lo = silu_mul(lo, ulo);
            hi = silu_mul(hi, uhi);
        }
        const int batch = (tile0 + nt) * kRowsPerTile + (t >> 1);
        const int r0 = out_tile * 16 + g;
        if (CHAIN && id_batch >= 0) {   // an indexed product keeps one activation row and stores it as its pair's row
            if ((t & 1) == 0 && batch == id_batch) store_result<EPI>(y, ldy, rows, id_out, r0, id_ok ? lo : 0.0f, id_ok ? hi : 0.0f, push);
        } else if ((t & 1) == 0 && batch < m) store_result<EPI>(y, ldy, rows, batch, r0, lo, hi, push);
    }
    if (CHAIN) {
        // this warp stored one 16-row tile of the result for every activation row; the warp that completes a 256-wide
        // block runs the block's job
        if (chain.job.kind != 0 && (out_tile >> 4) < chain.job.blocks) {
            // Pushed results need no fence: the job polls every pair's stamp, which is what tells it a value has landed
            // (a fence here would wait for the peers' acknowledgements over NVLink, microseconds per warp); the
            // ticket then only picks the warp that runs the job.
            if (!(EPI == kEpiPush && chain.job.kind == 3)) __threadfence();
            __syncwarp();
            unsigned seen = 0;
            if (lane == 0) seen = atomicAdd(chain.job.tickets + (out_tile >> 4), 1u);
            seen = __shfl_sync(0xffffffffu, seen, 0);
            if (seen == 15u) chain_job<EPI>(chain.job, out_tile >> 4, m, *reinterpret_cast<PrepSmem*>(warp_smem));
        }
    }
}

// Which row tile a warp works on.  Plain store: consecutive tiles.  SwiGLU: even warp-rows take
// gate tile `pair`, odd warp-rows the matching up tile `pair + ff_tiles` (gate rows are stacked
// first, crates/ferric-llama/src/qwen35.rs:431).
template <int EPI>
__device__ __forceinline__ void pick_tile(int wk, int row_tiles, int ff_tiles, int& rt, int& out_tile, bool& active)
{
    const int warp = threadIdx.x >> 5, wr = warp / wk, wr_count = 8 / wk;
    if (EPI != kEpiSwiglu) {
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
    uint4 q5;   // Q5_K only: the fifth bits of this lane's weights, bytes 0..7 row g, bytes 8..15 row g + 8
};
// Stage copy: the unit is mirrored byte for byte into the warp's ring slot.  Every lane copies its
// own four 16-byte quant chunks; lanes 0..15 also copy one header row each.
template <bool Q5 = false>
__device__ __forceinline__ void q4k_issue(uint8_t* slot, const uint8_t* units, size_t unit, int lane)
{
    const uint8_t* src = units + unit * (Q5 ? kQ5KUnit : kQ4KUnit);
    if (lane < 16) cp_async_16(slot + 16 * lane, src + 16 * lane);
#pragma unroll
    for (int s = 0; s < (Q5 ? 5 : 4); s++) cp_async_16(slot + 256 + 512 * s + 16 * lane, src + 256 + 512 * s + 16 * lane);
}
template <bool Q5 = false>
__device__ __forceinline__ void q4k_read(Q4KUnit& u, const uint8_t* slot, int lane)
{
    const uint4* p = reinterpret_cast<const uint4*>(slot);
    const int g = lane >> 2;
    u.hg = p[g];
    u.hh = p[8 + g];
#pragma unroll
    for (int s = 0; s < 4; s++) u.q[s] = p[16 + 32 * s + lane];
    if (Q5) u.q5 = p[16 + 32 * 4 + lane];
}

// 6-bit scales / mins of one row's super-block as clean bytes: sc[0..3], sc[4..7], m[0..3], m[4..7]
// (unpack rule: crates/ferric-gguf/src/lib.rs:795-804).
struct Q4KRow {
    uint32_t sc_lo, sc_hi, m_lo, m_hi;
    float d, dmin;
};
__device__ __forceinline__ void q4k_row(const uint4& h, Q4KRow& r)
{
    r.d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
    r.dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
    r.sc_lo = h.y & 0x3f3f3f3fu;
    r.m_lo = h.z & 0x3f3f3f3fu;
    r.sc_hi = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
    r.m_hi = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
}

// Q5 = true is the Q5_K kernel (crates/ferric-tensor/src/dtype.rs:1049-1071): the same product with 5-bit quants -- the
// fifth bit of each weight is OR-ed into its byte before the integer MMA; header, scales and mins are Q4_K's.
template <int NT, int EPI, bool Q5 = false, bool CHAIN = false>
__global__ void __launch_bounds__(256, NT <= 2 ? 2 : 1)
gemv_q4k_kernel(const uint8_t* __restrict__ units, const uint2* __restrict__ frag, float* __restrict__ y, int rows,
                int nblk, int m, size_t ldy, int row_tiles, int wk, int ff_tiles, PushDst push, Chain chain)
{
    __shared__ float red[8][NT * 4][32];
    constexpr int kUnitBytes = Q5 ? kQ5KUnit : kQ4KUnit;
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, t = lane & 3;
    int rt, out_tile;
    bool active;
    pick_tile<EPI>(wk, row_tiles, ff_tiles, rt, out_tile, active);
    const int kpart = warp % wk, per = (nblk + wk - 1) / wk;
    const int b0 = kpart * per, b1 = min(nblk, b0 + per);
    int tile0 = blockIdx.y * NT;
    const int zero[4] = {0, 0, 0, 0};
    IdPick idp;
    if (CHAIN && chain.id.selw) {
        // an indexed product learns its expert from the router's output, so nothing can be requested before the wait
        pdl_wait();
        idp = id_pick(chain.id);
        units += (size_t)idp.expert * (chain.id.rows_per_expert / 16) * nblk * kUnitBytes;
        tile0 = idp.batch / kRowsPerTile;
    }

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;

    // weights never change, so their first pipeline stages are requested before the wait on the
    // preceding kernel; everything that depends on the activations comes after it
    const bool work = active && b0 < b1;
    uint8_t* ring = gemv_smem + (size_t)warp * (kStagesQ4K * kUnitBytes);
    const uint8_t* wsrc = units + ((size_t)(work ? rt : 0) * nblk + (work ? b0 : 0)) * kUnitBytes;   // next unit to copy
    int issued = b0, wstage = 0, rstage = 0;
    if (work) {
#pragma unroll
        for (int i = 0; i < kStagesQ4K - 1; i++) {
            if (issued < b1) {
                q4k_issue<Q5>(ring + wstage * kUnitBytes, wsrc, 0, lane);
                wsrc += kUnitBytes;
                issued++;
                wstage = wstage + 1 == kStagesQ4K ? 0 : wstage + 1;
            }
            cp_async_commit();
        }
    }
    pdl_wait();
    float inv[NT];
    chain_scales<NT, CHAIN>(inv, chain, tile0, m);
    if (work) {
        const uint2* fsrc[NT];                                                 // fragments of the next unit to use
#pragma unroll
        for (int nt = 0; nt < NT; nt++) fsrc[nt] = frag + ((size_t)(tile0 + nt) * nblk + b0) * (kQ4KSteps * 32) + lane;
        constexpr bool kAhead = NT == 1;  // with more column tiles the second buffer would spill
        uint2 bf[NT][kQ4KSteps];
        if (kAhead) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int s = 0; s < kQ4KSteps; s++) bf[nt][s] = ld_act(fsrc[nt] + s * 32);
        }

        for (int b = b0; b < b1; b++) {
            if (issued < b1) {
                q4k_issue<Q5>(ring + wstage * kUnitBytes, wsrc, 0, lane);
                wsrc += kUnitBytes;
                issued++;
                wstage = wstage + 1 == kStagesQ4K ? 0 : wstage + 1;
            }
            cp_async_commit();
            uint2 bn[kAhead ? NT : 1][kQ4KSteps];
            if (kAhead) {
                if (b + 1 < b1) {
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        fsrc[nt] += kQ4KSteps * 32;
#pragma unroll
                        for (int s = 0; s < kQ4KSteps; s++) bn[nt][s] = ld_act(fsrc[nt] + s * 32);
                    }
                }
            } else {  // issue this super-block's fragment loads before waiting for its weights
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                    for (int s = 0; s < kQ4KSteps; s++) bf[nt][s] = ld_act(fsrc[nt] + s * 32);
                    fsrc[nt] += kQ4KSteps * 32;
                }
            }
            cp_async_wait<kStagesQ4K - 1>();
            __syncwarp();
            Q4KUnit cur;
            q4k_read<Q5>(cur, ring + rstage * kUnitBytes, lane);
            rstage = rstage + 1 == kStagesQ4K ? 0 : rstage + 1;
            __syncwarp();  // every lane has its copy before a later stage copy may overwrite the slot
            Q4KRow rg, rh;
            q4k_row(cur.hg, rg);
            q4k_row(cur.hh, rh);

            int ai[NT][4];  // sum_sb sc * (q . limb), per column
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++) ai[nt][i] = 0;

#pragma unroll
            for (int p = 0; p < 4; p++) {  // 32-byte group p: sub-blocks 2p (low nibbles), 2p+1 (high)
                const uint4 qg = cur.q[p >> 1], qh = cur.q[2 + (p >> 1)];
                const uint32_t w0 = (p & 1) ? qg.z : qg.x, w1 = (p & 1) ? qg.w : qg.y;
                const uint32_t v0 = (p & 1) ? qh.z : qh.x, v1 = (p & 1) ? qh.w : qh.y;
#pragma unroll
                for (int n = 0; n < 2; n++) {
                    const int s = 2 * p + n;
                    uint32_t a0 = (n ? (w0 >> 4) : w0) & 0x0f0f0f0fu, a2 = (n ? (w1 >> 4) : w1) & 0x0f0f0f0fu;
                    uint32_t a1 = (n ? (v0 >> 4) : v0) & 0x0f0f0f0fu, a3 = (n ? (v1 >> 4) : v1) & 0x0f0f0f0fu;
                    if (Q5) {   // bit s of the lane's eight qh bytes per row -> bit 4 of the matching weight byte
                        a0 |= ((cur.q5.x >> s) & 0x01010101u) << 4;
                        a2 |= ((cur.q5.y >> s) & 0x01010101u) << 4;
                        a1 |= ((cur.q5.z >> s) & 0x01010101u) << 4;
                        a3 |= ((cur.q5.w >> s) & 0x01010101u) << 4;
                    }
                    const int scg = (int)__byte_perm(s < 4 ? rg.sc_lo : rg.sc_hi, 0u, 0x4440u | (uint32_t)(s & 3));
                    const int sch = (int)__byte_perm(s < 4 ? rh.sc_lo : rh.sc_hi, 0u, 0x4440u | (uint32_t)(s & 3));
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        int c[4];
                        imma_16832_u8s8(c, a0, a1, a2, a3, bf[nt][s].x, bf[nt][s].y, zero);
                        ai[nt][0] += scg * c[0];
                        ai[nt][1] += scg * c[1];
                        ai[nt][2] += sch * c[2];
                        ai[nt][3] += sch * c[3];
                    }
                }
            }
            // mins: sum_sb m[sb] * (limb sum of sub-block sb); k slot 4t+i <-> sub-block 4t+i (0..7)
            const uint32_t mg = t == 0 ? rg.m_lo : t == 1 ? rg.m_hi : 0u;
            const uint32_t mh = t == 0 ? rh.m_lo : t == 1 ? rh.m_hi : 0u;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                int c0[4], c1[4];
                imma_16816_u8s8(c0, mg, mh, bf[nt][8].x, zero);
                imma_16816_u8s8(c1, mg, mh, bf[nt][8].y, zero);
                const float up = __uint_as_float(bf[nt][9].x);
                const float fg = rg.d * up, fmg = -rg.dmin * up, fh = rh.d * up, fmh = -rh.dmin * up;
                acc[nt][0] = fmaf(fmg, (float)(c0[0] + 128 * c1[0]), fmaf(fg, (float)ai[nt][0], acc[nt][0]));
                acc[nt][1] = fmaf(fmg, (float)(c0[1] + 128 * c1[1]), fmaf(fg, (float)ai[nt][1], acc[nt][1]));
                acc[nt][2] = fmaf(fmh, (float)(c0[2] + 128 * c1[2]), fmaf(fh, (float)ai[nt][2], acc[nt][2]));
                acc[nt][3] = fmaf(fmh, (float)(c0[3] + 128 * c1[3]), fmaf(fh, (float)ai[nt][3], acc[nt][3]));
            }
            if (kAhead) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int s = 0; s < kQ4KSteps; s++) bf[nt][s] = bn[nt][s];
            }
        }
    }
    reduce_and_store<NT, EPI, CHAIN>(acc, red, y, ldy, EPI == kEpiSwiglu ? rows / 2 : rows, m, tile0, wk, out_tile, active, push, inv,
                                     chain, ring, idp.batch, idp.out, idp.ok);
}

// ------------------------------------------------------------------------------------------
// Q6_K
// ------------------------------------------------------------------------------------------
struct Q6KUnit {
    uint32_t dpair;
    uint4 scg, sch, ql[4], qh[2];
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
    const int g = lane >> 2;
    u.dpair = *reinterpret_cast<const uint32_t*>(p + 4 * g);
    u.scg = *reinterpret_cast<const uint4*>(p + kQ6KOffSc + 16 * g);
    u.sch = *reinterpret_cast<const uint4*>(p + kQ6KOffSc + 16 * (g + 8));
#pragma unroll
    for (int s = 0; s < 4; s++) u.ql[s] = *reinterpret_cast<const uint4*>(p + kQ6KOffQl + 512 * s + 16 * lane);
#pragma unroll
    for (int s = 0; s < 2; s++) u.qh[s] = *reinterpret_cast<const uint4*>(p + kQ6KOffQh + 512 * s + 16 * lane);
}
__device__ __forceinline__ uint32_t u4_word(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
// sign-extended byte `i` (0..15) of a 16-byte scale row: PRMT copies the byte and replicates its
// sign bit into the three upper bytes (selector nibble 8|b)
__device__ __forceinline__ int sc_byte(const uint4& v, int i)
{
    const uint32_t b = (uint32_t)(i & 3);
    const uint32_t sel = b | ((8u | b) << 4) | ((8u | b) << 8) | ((8u | b) << 12);
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(u4_word(v, i >> 2)), "r"(0u), "r"(sel));
    return (int)d;
}

// One unit (16 rows x one super-block) times the prepared activation fragments of NT tiles: integer sub-block sums
// scaled by the int8 sub-block scales, the -32 offset taken off through the fragments' sub-block sums, then d and the
// activation block scale in f32.
template <int NT>
__device__ __forceinline__ void q6k_unit_mac(const Q6KUnit& cur, const uint2 (&bf)[NT][kQ6KSteps], float (&acc)[NT][4], int t)
{
    const int zero[4] = {0, 0, 0, 0};
    int ai[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) ai[nt][i] = 0;

#pragma unroll
    for (int h = 0; h < 2; h++) {
#pragma unroll
        for (int k = 0; k < 4; k++) {
            // double step 4h + k: sub-blocks sb = 8h + 2k + is, is = 0 (.x) and 1 (.y)
#pragma unroll
            for (int is = 0; is < 2; is++) {
                const int wi = 2 * h + is, sb = 8 * h + 2 * k + is;
                // 6-bit weights of rows g and g+8: low nibble source word, high-bit source word
                const uint32_t lg = u4_word(cur.ql[k & 1], wi), lh = u4_word(cur.ql[2 + (k & 1)], wi);
                const uint32_t hg = u4_word(cur.qh[0], wi), hh = u4_word(cur.qh[1], wi);
                const uint32_t lo_g = ((k & 2) ? (lg >> 4) : lg) & 0x0f0f0f0fu;
                const uint32_t lo_h = ((k & 2) ? (lh >> 4) : lh) & 0x0f0f0f0fu;
                const uint32_t hi_g = (k == 0 ? (hg << 4) : k == 1 ? (hg << 2) : k == 2 ? hg : (hg >> 2)) & 0x30303030u;
                const uint32_t hi_h = (k == 0 ? (hh << 4) : k == 1 ? (hh << 2) : k == 2 ? hh : (hh >> 2)) & 0x30303030u;
                const uint32_t a0 = lo_g | hi_g, a1 = lo_h | hi_h;
                const int scg = sc_byte(cur.scg, sb), sch = sc_byte(cur.sch, sb);
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    int c[4];
                    imma_16816_u8s8(c, a0, a1, is ? bf[nt][4 * h + k].y : bf[nt][4 * h + k].x, zero);
                    ai[nt][0] += scg * c[0];
                    ai[nt][1] += scg * c[1];
                    ai[nt][2] += sch * c[2];
                    ai[nt][3] += sch * c[3];
                }
            }
        }
    }
    // the -32 offset: sum_sb sc[sb] * (limb sum of sub-block sb); k slot 4t+i <-> sub-block 4t+i
    const uint32_t sg = u4_word(cur.scg, t), sh = u4_word(cur.sch, t);
    const float dg = __half2float(__ushort_as_half((unsigned short)(cur.dpair & 0xffffu)));
    const float dh = __half2float(__ushort_as_half((unsigned short)(cur.dpair >> 16)));
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        int c0[4], c1[4];
        imma_16816_s8s8(c0, sg, sh, bf[nt][8].x, zero);
        imma_16816_s8s8(c1, sg, sh, bf[nt][8].y, zero);
        const float up = __uint_as_float(bf[nt][9].x);
        const float fg = dg * up, fh = dh * up;
        acc[nt][0] = fmaf(fg, (float)(ai[nt][0] - 32 * (c0[0] + 128 * c1[0])), acc[nt][0]);
        acc[nt][1] = fmaf(fg, (float)(ai[nt][1] - 32 * (c0[1] + 128 * c1[1])), acc[nt][1]);
        acc[nt][2] = fmaf(fh, (float)(ai[nt][2] - 32 * (c0[2] + 128 * c1[2])), acc[nt][2]);
        acc[nt][3] = fmaf(fh, (float)(ai[nt][3] - 32 * (c0[3] + 128 * c1[3])), acc[nt][3]);
    }
}

template <int NT, int EPI, bool CHAIN = false>
__global__ void __launch_bounds__(256, NT <= 2 ? 2 : 1)
gemv_q6k_kernel(const uint8_t* __restrict__ units, const uint2* __restrict__ frag, float* __restrict__ y, int rows,
                int nblk, int m, size_t ldy, int row_tiles, int wk, int ff_tiles, PushDst push, Chain chain)
{
    __shared__ float red[8][NT * 4][32];
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, t = lane & 3;
    int rt, out_tile;
    bool active;
    pick_tile<EPI>(wk, row_tiles, ff_tiles, rt, out_tile, active);
    const int kpart = warp % wk, per = (nblk + wk - 1) / wk;
    const int b0 = kpart * per, b1 = min(nblk, b0 + per);
    int tile0 = blockIdx.y * NT;
    IdPick idp;
    if (CHAIN && chain.id.selw) {
        // an indexed product learns its expert from the router's output, so nothing can be requested before the wait
        pdl_wait();
        idp = id_pick(chain.id);
        units += (size_t)idp.expert * (chain.id.rows_per_expert / 16) * nblk * kQ6KUnit;
        tile0 = idp.batch / kRowsPerTile;
    }

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;

    // weights never change, so their first pipeline stages are requested before the wait on the
    // preceding kernel; everything that depends on the activations comes after it
    const bool work = active && b0 < b1;
    uint8_t* ring = gemv_smem + (size_t)warp * (kStagesQ6K * kQ6KUnit);
    const uint8_t* wsrc = units + ((size_t)(work ? rt : 0) * nblk + (work ? b0 : 0)) * kQ6KUnit;   // next unit to copy
    int issued = b0, wstage = 0, rstage = 0;
    if (work) {
#pragma unroll
        for (int i = 0; i < kStagesQ6K - 1; i++) {
            if (issued < b1) {
                q6k_issue(ring + wstage * kQ6KUnit, wsrc, 0, lane);
                wsrc += kQ6KUnit;
                issued++;
                wstage = wstage + 1 == kStagesQ6K ? 0 : wstage + 1;
            }
            cp_async_commit();
        }
    }
    pdl_wait();
    float inv[NT];
    chain_scales<NT, CHAIN>(inv, chain, tile0, m);
    if (work) {
        const uint2* fsrc[NT];                                                 // fragments of the next unit to use
#pragma unroll
        for (int nt = 0; nt < NT; nt++) fsrc[nt] = frag + ((size_t)(tile0 + nt) * nblk + b0) * (kQ6KSteps * 32) + lane;
        constexpr bool kAhead = NT == 1;
        uint2 bf[NT][kQ6KSteps];
        if (kAhead) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int s = 0; s < kQ6KSteps; s++) bf[nt][s] = ld_act(fsrc[nt] + s * 32);
        }
        for (int b = b0; b < b1; b++) {
            if (issued < b1) {
                q6k_issue(ring + wstage * kQ6KUnit, wsrc, 0, lane);
                wsrc += kQ6KUnit;
                issued++;
                wstage = wstage + 1 == kStagesQ6K ? 0 : wstage + 1;
            }
            cp_async_commit();
            uint2 bn[kAhead ? NT : 1][kQ6KSteps];
            if (kAhead) {
                if (b + 1 < b1) {
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        fsrc[nt] += kQ6KSteps * 32;
#pragma unroll
                        for (int s = 0; s < kQ6KSteps; s++) bn[nt][s] = ld_act(fsrc[nt] + s * 32);
                    }
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                    for (int s = 0; s < kQ6KSteps; s++) bf[nt][s] = ld_act(fsrc[nt] + s * 32);
                    fsrc[nt] += kQ6KSteps * 32;
                }
            }
            cp_async_wait<kStagesQ6K - 1>();
            __syncwarp();
            Q6KUnit cur;
            q6k_read(cur, ring + rstage * kQ6KUnit, lane);
            rstage = rstage + 1 == kStagesQ6K ? 0 : rstage + 1;
            __syncwarp();

            q6k_unit_mac<NT>(cur, bf, acc, t);
            if (kAhead) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int s = 0; s < kQ6KSteps; s++) bf[nt][s] = bn[nt][s];
            }
        }
    }
    reduce_and_store<NT, EPI, CHAIN>(acc, red, y, ldy, EPI == kEpiSwiglu ? rows / 2 : rows, m, tile0, wk, out_tile, active, push, inv,
                                     chain, ring, idp.batch, idp.out, idp.ok);
}

// ------------------------------------------------------------------------------------------
// Q6_K, unit-balanced: the matrix's units (row tile major, super-block minor -- the order they lie in memory) are
// dealt out evenly to all resident warps, so a warp streams one contiguous byte range whatever the shape, and the
// machine is equally loaded even when the row tiles do not fill a whole number of waves.  A warp's range may start
// and end inside a row tile; such partial sums go to the workspace and the last warp to arrive at a tile (a ticket
// per tile) adds the tile's pieces in warp order -- a fixed order, so results do not depend on timing.
// Off by default (FERRIC_CUDA_GEMV_STREAM=1 turns it on): on the 5120 x 17408 down projection it measured the same
// 22 us as the row-tile form, whose 320 CTAs leave a part-filled second wave -- the kernel is bound by instruction
// issue (about 360 instructions per unit, issue slots half used), not by how evenly the units are dealt.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned stream_first_unit(unsigned long long units, unsigned w, unsigned warps)
{
    return (unsigned)(units * w / warps);
}
__device__ __forceinline__ unsigned stream_warp_of(unsigned long long units, unsigned unit, unsigned warps)
{
    return (unsigned)((((unsigned long long)unit + 1) * warps - 1) / units);   // the largest w with first_unit(w) <= unit
}

template <int NT, int EPI>
__global__ void __launch_bounds__(256, NT <= 2 ? 2 : 1)
gemv_q6k_stream_kernel(const uint8_t* __restrict__ units, const uint2* __restrict__ frag, float* __restrict__ y, int rows,
                       int nblk, int m, size_t ldy, int row_tiles, PushDst push, SplitWs split)
{
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const unsigned warps = gridDim.x * 8, w = blockIdx.x * 8 + warp;
    const unsigned long long total = (unsigned long long)row_tiles * nblk;
    const unsigned u0 = stream_first_unit(total, w, warps), u1 = stream_first_unit(total, w + 1, warps);
    const int tile0 = blockIdx.y * NT;

    uint8_t* ring = gemv_smem + (size_t)warp * (kStagesQ6K * kQ6KUnit);
    const uint8_t* wsrc = units + (size_t)u0 * kQ6KUnit;   // next unit to copy: the range is contiguous in memory
    unsigned issued = u0;
    int wstage = 0, rstage = 0;
#pragma unroll
    for (int i = 0; i < kStagesQ6K - 1; i++) {
        if (issued < u1) {
            q6k_issue(ring + wstage * kQ6KUnit, wsrc, 0, lane);
            wsrc += kQ6KUnit;
            issued++;
            wstage = wstage + 1 == kStagesQ6K ? 0 : wstage + 1;
        }
        cp_async_commit();
    }
    pdl_wait();
    if (u0 >= u1) return;

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;
    int tile = (int)(u0 / (unsigned)nblk), b = (int)(u0 % (unsigned)nblk), seg_b0 = b;
    const float w0 = (t & 1) ? 6.103515625e-05f : 1.0f;            // limb weights, as in reduce_and_store
    const float w1 = (t & 1) ? 4.76837158203125e-07f : 0.0078125f;
    float* my_slots = split.partial + ((size_t)blockIdx.y * warps + w) * 2 * (NT * 64);
    constexpr bool kAhead = NT == 1;
    uint2 bf[NT][kQ6KSteps];
    if (kAhead) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint2* fsrc = frag + ((size_t)(tile0 + nt) * nblk + b) * (kQ6KSteps * 32) + lane;
#pragma unroll
            for (int s = 0; s < kQ6KSteps; s++) bf[nt][s] = ld_act(fsrc + s * 32);
        }
    }

    for (unsigned u = u0; u < u1; u++) {
        if (issued < u1) {
            q6k_issue(ring + wstage * kQ6KUnit, wsrc, 0, lane);
            wsrc += kQ6KUnit;
            issued++;
            wstage = wstage + 1 == kStagesQ6K ? 0 : wstage + 1;
        }
        cp_async_commit();
        // activation fragments: with one tile they are fetched one unit ahead (the fragments depend on the super-block
        // only, so the one after the last of a row tile is the first again)
        uint2 bn[kAhead ? NT : 1][kQ6KSteps];
        if (kAhead) {
            if (u + 1 < u1) {
                const int nb = b + 1 == nblk ? 0 : b + 1;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const uint2* fsrc = frag + ((size_t)(tile0 + nt) * nblk + nb) * (kQ6KSteps * 32) + lane;
#pragma unroll
                    for (int s = 0; s < kQ6KSteps; s++) bn[nt][s] = ld_act(fsrc + s * 32);
                }
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint2* fsrc = frag + ((size_t)(tile0 + nt) * nblk + b) * (kQ6KSteps * 32) + lane;
#pragma unroll
                for (int s = 0; s < kQ6KSteps; s++) bf[nt][s] = ld_act(fsrc + s * 32);
            }
        }
        cp_async_wait<kStagesQ6K - 1>();
        __syncwarp();
        Q6KUnit cur;
        q6k_read(cur, ring + rstage * kQ6KUnit, lane);
        rstage = rstage + 1 == kStagesQ6K ? 0 : rstage + 1;
        __syncwarp();
        q6k_unit_mac<NT>(cur, bf, acc, t);
        if (kAhead) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int s = 0; s < kQ6KSteps; s++) bf[nt][s] = bn[nt][s];
        }
        b++;
        if (b < nblk && u + 1 < u1) continue;

        // ---- the segment [seg_b0, b) of row tile `tile` ends here
        const bool whole = seg_b0 == 0 && b == nblk;
        const int r0 = tile * 16 + g;
        float lo[NT], hi[NT];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            lo[nt] = acc[nt][0] * w0 + acc[nt][1] * w1;
            hi[nt] = acc[nt][2] * w0 + acc[nt][3] * w1;
            lo[nt] += __shfl_xor_sync(0xffffffffu, lo[nt], 1);
            hi[nt] += __shfl_xor_sync(0xffffffffu, hi[nt], 1);
#pragma unroll
            for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;
        }
        if (whole) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int batch = (tile0 + nt) * kRowsPerTile + (t >> 1);
                if ((t & 1) == 0 && batch < m) store_result<EPI>(y, ldy, rows, batch, r0, lo[nt], hi[nt], push);
            }
        } else {
            // slot 0: a piece that starts inside the tile (only a warp's first piece can); slot 1: one that starts with it
            float* slot = my_slots + (seg_b0 > 0 ? 0 : 1) * (NT * 64);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) __stcg(reinterpret_cast<float2*>(slot + nt * 64) + lane, make_float2(lo[nt], hi[nt]));
            __threadfence();
            __syncwarp();
            const unsigned t_first = (unsigned)tile * (unsigned)nblk, t_last = t_first + (unsigned)nblk - 1;
            const unsigned w_lo = stream_warp_of(total, t_first, warps), w_hi = stream_warp_of(total, t_last, warps);
            unsigned seen = 0;
            unsigned* ticket = split.tickets + (size_t)blockIdx.y * row_tiles + tile;
            if (lane == 0) seen = atomicAdd(ticket, 1u);
            seen = __shfl_sync(0xffffffffu, seen, 0);
            if (seen == w_hi - w_lo) {   // every other piece of this tile is in the workspace: add them in warp order
                __threadfence();
                float slo[NT], shi[NT];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) slo[nt] = shi[nt] = 0.0f;
                for (unsigned ww = w_lo; ww <= w_hi; ww++) {
                    const unsigned s0 = stream_first_unit(total, ww, warps);
                    const float* src = split.partial + (((size_t)blockIdx.y * warps + ww) * 2 + (s0 > t_first ? 0 : 1)) * (NT * 64);
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const float2 v = __ldcg(reinterpret_cast<const float2*>(src + nt * 64) + lane);
                        slo[nt] += v.x;
                        shi[nt] += v.y;
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int batch = (tile0 + nt) * kRowsPerTile + (t >> 1);
                    if ((t & 1) == 0 && batch < m) store_result<EPI>(y, ldy, rows, batch, r0, slo[nt], shi[nt], push);
                }
                if (lane == 0) *ticket = 0;   // ready for the next launch
            }
        }
        tile++;
        b = 0;
        seg_b0 = 0;
    }
}

// ------------------------------------------------------------------------------------------
// launch
// ------------------------------------------------------------------------------------------
// How many of a CTA's 8 warps split K (the rest take different row tiles).  The grid should fit
// in as few waves of resident CTAs as possible -- every wave pays its own pipeline fill and
// drain -- and within that, K-splitting shortens each warp's serial walk.  Cost model: waves x
// (super-blocks per warp + a fixed fill/drain term), measured in super-block times.
static int choose_wk(uint32_t ty, const DeviceWeights& w, Epilogue epi, int nt, const GemvTuning& tune)
{
    int forced = tune.wk;
    const int ctas_per_sm = nt <= 2 ? 2 : 1;
    const size_t slots = (size_t)tune.sm_count * ctas_per_sm;
    const size_t tiles = epi == kEpiSwiglu ? w.rows / 2 / 16 * 2 : w.row_tiles();
    int best = 1;
    double best_cost = 1e30;
    for (int wk = 1; wk <= 8; wk *= 2) {
        if ((size_t)wk > w.nblk && wk > 1) break;
        if (epi == kEpiSwiglu && wk > 4) break;
        if (forced == wk) return wk;
        const size_t ctas = (tiles + (size_t)(8 / wk) - 1) / (size_t)(8 / wk);
        // Q6_K's ring is a stage shallower and a CTA alone on an SM does not keep enough loads in flight, so for it a
        // part-filled second wave is charged its share rather than a whole wave
        // (measured on the 5120 x 17408 down projection: 22.2 us with 320 CTAs against 23.3 us with 160)
        const double waves = ty == kGgmlQ6K ? ((double)ctas > (double)slots ? (double)ctas / (double)slots : 1.0)
                                            : (double)((ctas + slots - 1) / slots);
        const double cost = waves * ((double)((w.nblk + wk - 1) / wk) + 4.0);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = wk;
        }
    }
    return best;
}

template <int NT, int EPI, bool CHAIN>
static void launch_gemv_t(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const uint2* frag, size_t m, float* y,
                          size_t ldy, int wk, unsigned passes, bool pdl, const PushDst& push, const SplitWs& split,
                          bool stream, int stream_ctas, int sm_count, const Chain& chain)
{
    const int row_tiles = (int)w.row_tiles(), wr = 8 / wk;
    const int ff_tiles = (int)(w.rows / 2 / 16);
    unsigned gx = EPI != kEpiSwiglu ? (unsigned)((row_tiles + wr - 1) / wr) : (unsigned)((ff_tiles + wr / 2 - 1) / (wr / 2));
    dim3 grid(gx, passes);
    // opt in to > 48 KB of dynamic shared memory once per kernel instantiation and device
    static thread_local int attr_dev_q4 = -1, attr_dev_q6 = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (ty == kGgmlQ4K) {
        if (attr_dev_q4 != dev) {
            cudaFuncSetAttribute(gemv_q4k_kernel<NT, EPI, false, CHAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemQ4K);
            attr_dev_q4 = dev;
        }
        launch_kernel(gemv_q4k_kernel<NT, EPI, false, CHAIN>, grid, dim3(256), kSmemQ4K, st, pdl, w.units, frag, y, (int)w.rows,
                      (int)w.nblk, (int)m, ldy, row_tiles, wk, ff_tiles, push, chain);
    } else if (ty == kGgmlQ5K) {
        static thread_local int attr_dev_q5 = -1;
        if (attr_dev_q5 != dev) {
            cudaFuncSetAttribute(gemv_q4k_kernel<NT, EPI, true, CHAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemQ5K);
            attr_dev_q5 = dev;
        }
        launch_kernel(gemv_q4k_kernel<NT, EPI, true, CHAIN>, grid, dim3(256), kSmemQ5K, st, pdl, w.units, frag, y, (int)w.rows,
                      (int)w.nblk, (int)m, ldy, row_tiles, wk, ff_tiles, push, chain);
    } else {
        if (attr_dev_q6 != dev) {
            cudaFuncSetAttribute(gemv_q6k_kernel<NT, EPI, CHAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemQ6K);
            if (EPI != kEpiSwiglu && !CHAIN)
                cudaFuncSetAttribute(gemv_q6k_stream_kernel<NT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemQ6K);
            attr_dev_q6 = dev;
        }
        if constexpr (EPI != kEpiSwiglu && !CHAIN) {
            // the unit-balanced form: one resident CTA per slot, every warp an equal share of the units
            const unsigned ctas = stream_ctas > 0 ? (unsigned)stream_ctas : (unsigned)sm_count * (NT <= 2 ? 2u : 1u);
            const size_t total = (size_t)row_tiles * w.nblk, warps = (size_t)ctas * 8;
            if (stream && split.partial && passes == 1 && total >= warps && (size_t)row_tiles <= kSplitTickets &&
                warps * 2 * NT * 64 <= kSplitWsFloats) {
                launch_kernel(gemv_q6k_stream_kernel<NT, EPI>, dim3(ctas, passes), dim3(256), kSmemQ6K, st, pdl, w.units, frag, y,
                              (int)w.rows, (int)w.nblk, (int)m, ldy, row_tiles, push, split);
                return;
            }
        }
        launch_kernel(gemv_q6k_kernel<NT, EPI, CHAIN>, grid, dim3(256), kSmemQ6K, st, pdl, w.units, frag, y, (int)w.rows,
                      (int)w.nblk, (int)m, ldy, row_tiles, wk, ff_tiles, push, chain);
    }
}

int32_t launch_gemv(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const void* frag, size_t m, float* y,
                    size_t ldy, Epilogue epi, const GemvTuning& tune, const PushDst& push, const Chain* chain)
{
    if (m == 0 || w.rows == 0) return kOk;
    const int nt = tiles_per_pass(m), wk = choose_wk(ty, w, epi, nt, tune);
    const unsigned passes = (unsigned)(padded_tiles(m) / (size_t)nt);
    const uint2* f = reinterpret_cast<const uint2*>(frag);
    if (chain && passes != 1) {
        set_last_error("a chained product takes at most %zu activation rows", kChainMaxRows);
        return kErrShape;
    }
    const Chain none;
#define FERRIC_GEMV_CASE2(NT_, CH_, ARG_)                                                                 \
    if (epi == kEpiStore) launch_gemv_t<NT_, kEpiStore, CH_>(st, ty, w, f, m, y, ldy, wk, passes, tune.pdl, push, tune.split_ws, tune.stream, tune.stream_ctas, tune.sm_count, ARG_);   \
    else if (epi == kEpiPush) launch_gemv_t<NT_, kEpiPush, CH_>(st, ty, w, f, m, y, ldy, wk, passes, tune.pdl, push, tune.split_ws, tune.stream, tune.stream_ctas, tune.sm_count, ARG_); \
    else launch_gemv_t<NT_, kEpiSwiglu, CH_>(st, ty, w, f, m, y, ldy, wk, passes, tune.pdl, push, tune.split_ws, tune.stream, tune.stream_ctas, tune.sm_count, ARG_)
#define FERRIC_GEMV_CASE(NT_)                         \
    if (chain) { FERRIC_GEMV_CASE2(NT_, true, *chain); } \
    else { FERRIC_GEMV_CASE2(NT_, false, none); }
    if (nt == 1) { FERRIC_GEMV_CASE(1) }
    else { FERRIC_GEMV_CASE(2) }
#undef FERRIC_GEMV_CASE
#undef FERRIC_GEMV_CASE2
    FERRIC_CUDA_TRY(cudaGetLastError());
    return kOk;
}

// Indexed products (crates/ferric-tensor/src/dtype.rs:1620-1677): one launch pass per (token, expert slot) pair over the
// selected expert's rows, one activation tile per pass.
int32_t launch_gemv_id(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const void* frag, size_t m, size_t pairs, float* y,
                       size_t ldy, Epilogue epi, const GemvTuning& tune, const IdSel& id)
{
    if (pairs == 0 || id.rows_per_expert == 0) return kOk;
    if (pairs > 65535) {
        set_last_error("an indexed product takes at most 65535 (token, expert) pairs per call (%zu given)", pairs);
        return kErrShape;
    }
    // the launch sees one expert's sub-matrix; the kernel moves the base to the pair's expert
    DeviceWeights one = w;
    one.rows = (size_t)id.rows_per_expert;
    Chain chain;
    chain.id = id;
    const int wk = choose_wk(ty, one, epi, 1, tune);
    const uint2* f = reinterpret_cast<const uint2*>(frag);
    const PushDst none;
    if (epi == kEpiSwiglu)
        launch_gemv_t<1, kEpiSwiglu, true>(st, ty, one, f, m, y, ldy, wk, (unsigned)pairs, tune.pdl, none, tune.split_ws, false, 0, tune.sm_count, chain);
    else
        launch_gemv_t<1, kEpiStore, true>(st, ty, one, f, m, y, ldy, wk, (unsigned)pairs, tune.pdl, none, tune.split_ws, false, 0, tune.sm_count, chain);
    FERRIC_CUDA_TRY(cudaGetLastError());
    return kOk;
}

__global__ void id_wsum_kernel(const float* __restrict__ part, const float* __restrict__ selw, size_t t, size_t k, size_t out_pe,
                               float* __restrict__ out)
{
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = t * out_pe;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t ti = i / out_pe, o = i - ti * out_pe;
        float tot = 0.0f;
        for (size_t s = 0; s < k; s++) tot = tot + selw[ti * 2 * k + s] * part[(ti * k + s) * out_pe + o];   // slot order, as the reference sums
        out[i] = tot;
    }
}

int32_t launch_id_wsum(cudaStream_t st, const float* part, const float* selw, size_t t, size_t k, size_t out_pe, float* out,
                       const GemvTuning& tune)
{
    const size_t total = t * out_pe;
    if (total == 0) return kOk;
    size_t g = (total + 255) / 256;
    if (g > 148 * 16) g = 148 * 16;
    FERRIC_CUDA_TRY(launch_kernel(id_wsum_kernel, dim3((unsigned)g), dim3(256), 0, st, tune.pdl, part, selw, t, k, out_pe, out));
    return kOk;
}

// ------------------------------------------------------------------------------------------
// Q8_0: a warp owns kQ8Rows consecutive output rows; lanes stride 16-weight runs of K.  A lane loads its 16 activations
// of a run once into registers and uses them for all the warp's rows (one activation row at a time when there are
// several), so the activation traffic through L1 is 1/kQ8Rows of the weight traffic instead of four times it.  Each
// 16-weight half of a 32-weight block is summed in f32 and scaled by the block's d (crates/ferric-tensor/src/cpu_simd.rs:
// 57-72 scales per block); the lanes' partial sums meet in a warp-shuffle reduction.
// ------------------------------------------------------------------------------------------
constexpr int kQ8Rows = 8;
__global__ void __launch_bounds__(256) gemv_q8_0_kernel(const int8_t* __restrict__ qs, const uint16_t* __restrict__ dpl,
                                                        const float* __restrict__ x, int m, size_t ldx,
                                                        float* __restrict__ y, size_t ldy, int rows, int cols)
{
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = (blockIdx.x * 8 + warp) * kQ8Rows;
    if (row0 >= rows) return;
    const int nchunks = cols / 16, nb = cols / 32;
    for (int batch = blockIdx.y; batch < m; batch += gridDim.y) {
        float acc[kQ8Rows];
#pragma unroll
        for (int r = 0; r < kQ8Rows; r++) acc[r] = 0.0f;
        const float* xrow = x + (size_t)batch * ldx;
        // two runs per lane and trip, all their weight loads issued before the first use: bytes in flight are what this
        // kernel lives on (a row is only 10 runs per lane at 5120 columns)
        for (int c0 = lane; c0 < nchunks; c0 += 64) {
            uint4 wv[2][kQ8Rows];
            float dv[2][kQ8Rows];
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int c = c0 + 32 * u;
#pragma unroll
                for (int r = 0; r < kQ8Rows; r++) {
                    const int row = row0 + r;
                    wv[u][r] = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);   // int8 zeros after the sign flip below
                    dv[u][r] = 0.0f;
                    if (row < rows && c < nchunks) {
                        wv[u][r] = ld_stream_u4(qs + (size_t)row * cols + 16 * c);
                        dv[u][r] = __half2float(__ushort_as_half(dpl[(size_t)row * nb + (c >> 1)]));
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int c = c0 + 32 * u;
                if (c >= nchunks) break;
                float xv[16];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float4 f = ld_act(reinterpret_cast<const float4*>(xrow + 16 * c) + k);
                    xv[4 * k] = f.x; xv[4 * k + 1] = f.y; xv[4 * k + 2] = f.z; xv[4 * k + 3] = f.w;
                }
#pragma unroll
                for (int r = 0; r < kQ8Rows; r++) {
                    const uint32_t ww[4] = {wv[u][r].x ^ 0x80808080u, wv[u][r].y ^ 0x80808080u, wv[u][r].z ^ 0x80808080u,
                                            wv[u][r].w ^ 0x80808080u};
                    float part = 0.0f;
                    // int8 -> f32 without the conversion unit: the sign-flipped byte (0..255) dropped into the mantissa of
                    // 2^23 by a byte permute, minus 2^23 + 128 -- exact
#pragma unroll
                    for (int k = 0; k < 4; k++)
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            part = fmaf(xv[4 * k + j], __uint_as_float(__byte_perm(ww[k], 0x4B000000u, 0x7650 + j)) - 8388736.0f, part);
                    acc[r] = fmaf(part, dv[u][r], acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < kQ8Rows; r++) {
            float v = acc[r];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && row0 + r < rows) y[(size_t)batch * ldy + row0 + r] = v;
        }
    }
}

int32_t launch_gemv_q8_0(cudaStream_t st, const DeviceWeights& w, const float* x, size_t m, size_t ldx, float* y,
                         size_t ldy, const GemvTuning& tune)
{
    if (m == 0 || w.rows == 0) return kOk;
    // one grid row of CTAs per activation row up to 8, beyond that each CTA walks several (the weights of its 64 rows
    // then come from L1 / L2)
    dim3 grid((unsigned)((w.rows + 8 * kQ8Rows - 1) / (8 * kQ8Rows)), (unsigned)(m < 8 ? m : 8));
    FERRIC_CUDA_TRY(launch_kernel(gemv_q8_0_kernel, grid, dim3(256), 0, st, tune.pdl, w.q8_qs, w.q8_d, x, (int)m, ldx, y,
                                  ldy, (int)w.rows, (int)w.cols));
    return kOk;
}

// Dense f32 weights (QMatrix::from_dense, crates/ferric-tensor/src/dtype.rs:912-926: the fallback for formats without a
// packed kernel, which the loader dequantises): one warp per output row, 128-bit loads, warp-shuffle reduction.
template <int MB>
__global__ void __launch_bounds__(256) gemv_f32_kernel(const float* __restrict__ w, const float* __restrict__ x, int m, size_t ldx,
                                                       float* __restrict__ y, size_t ldy, int rows, int cols)
{
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 8 + warp;
    if (row >= rows) return;
    const int batch0 = blockIdx.y * MB;
    float acc[MB];
#pragma unroll
    for (int i = 0; i < MB; i++) acc[i] = 0.0f;
    const float* wrow = w + (size_t)row * cols;
    const int nvec = ((reinterpret_cast<uintptr_t>(wrow) & 15) == 0) ? cols / 4 : 0;   // rows of an odd length are not all 16-byte aligned
    for (int c = lane; c < nvec; c += 32) {
        const uint4 wb = ld_stream_u4(wrow + 4 * c);
        const float w0 = __uint_as_float(wb.x), w1 = __uint_as_float(wb.y), w2 = __uint_as_float(wb.z), w3 = __uint_as_float(wb.w);
#pragma unroll
        for (int i = 0; i < MB; i++) {
            if (batch0 + i >= m) break;
            const float4 xv = ld_act(reinterpret_cast<const float4*>(x + (size_t)(batch0 + i) * ldx) + c);
            acc[i] = fmaf(xv.w, w3, fmaf(xv.z, w2, fmaf(xv.y, w1, fmaf(xv.x, w0, acc[i]))));
        }
    }
    for (int c = 4 * nvec + lane; c < cols; c += 32) {
        const float wv = wrow[c];
#pragma unroll
        for (int i = 0; i < MB; i++)
            if (batch0 + i < m) acc[i] = fmaf(x[(size_t)(batch0 + i) * ldx + c], wv, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < MB; i++) {
        float v = acc[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && batch0 + i < m) y[(size_t)(batch0 + i) * ldy + row] = v;
    }
}

int32_t launch_gemv_f32(cudaStream_t st, const DeviceWeights& w, const float* x, size_t m, size_t ldx, float* y, size_t ldy,
                        const GemvTuning& tune)
{
    if (m == 0 || w.rows == 0) return kOk;
    dim3 grid((unsigned)((w.rows + 7) / 8), (unsigned)((m + 3) / 4));
    FERRIC_CUDA_TRY(launch_kernel(gemv_f32_kernel<4>, grid, dim3(256), 0, st, tune.pdl, w.dense, x, (int)m, ldx, y, ldy, (int)w.rows,
                                  (int)w.cols));
    return kOk;
}

// out[r, c] = silu(gu[r, c]) * gu[r, d + c]   (crates/ferric-tensor/src/lib.rs:2603-2618)
__global__ void swiglu_kernel(const float* __restrict__ gu, size_t t, size_t d, float* __restrict__ out)
{
    pdl_launch_dependents();
    pdl_wait();
    size_t total = t * d;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t r = i / d, c = i % d;
        out[i] = silu_mul(gu[r * 2 * d + c], gu[r * 2 * d + d + c]);
    }
}

int32_t launch_swiglu(cudaStream_t st, const float* gu, size_t t, size_t d, float* out, const GemvTuning& tune)
{
    size_t total = t * d;
    if (total == 0) return kOk;
    size_t g = (total + 255) / 256;
    if (g > 148 * 32) g = 148 * 32;
    FERRIC_CUDA_TRY(launch_kernel(swiglu_kernel, dim3((unsigned)g), dim3(256), 0, st, tune.pdl, gu, t, d, out));
    return kOk;
}

}  // namespace ferric
