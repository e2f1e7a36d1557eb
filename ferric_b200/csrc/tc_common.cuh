// tcgen05 / TMA / mbarrier wrappers and small helpers shared by the tensor-core kernels (prefill GEMM and the
// batched decode product).  Inline PTX for sm_100a; every wait is bounded.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace ferric {

constexpr unsigned long long kTcWaitNs = 1000000000ull;   // every mbarrier wait gives up after one second

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false if it did not complete within kTcWaitNs.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    const uint32_t a = smem_u32(bar);
    uint64_t t0 = 0;
    for (uint32_t i = 0;; i++) {
        uint32_t ok;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((i & 255u) == 255u) {
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > kTcWaitNs) return false;
        }
    }
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
// Cluster-wide address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar)
{
    // CTA-scope release as for a local arrive: what the leader's tensor core reads from this CTA's shared memory was
    // already handed to the async proxy by fence.proxy.async; a cluster-scope release here costs most of a microsecond.
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
// TMA load inside a CTA pair: the data lands in this CTA's shared memory, the completion bytes are counted on
// a barrier that may live in the pair's leader.  No multicast: every CTA fetches its own half.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
                 : "memory");
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);          // start address
    d |= (uint64_t)1 << 16;                           // leading-dimension offset: unused with a swizzle, kept at 1
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride between 8-row groups
    d |= (uint64_t)1 << 46;                           // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                           // SWIZZLE_128B
    return d;
}
// kind::f16, bf16 x bf16 -> f32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same MMA with the shared-memory descriptors given by their low words only (address field | leading-dimension
// field); the high word is the same for every 128-byte-swizzled K-major tile.  The issuing thread's instruction stream
// is the critical path of the narrow-tile kernels, so the per-MMA arithmetic is one 32-bit add per operand:
// advancing a descriptor by b bytes adds b >> 4 to its low word.
constexpr uint32_t kUmmaDescHiSw128 = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
__device__ __forceinline__ void umma_f16_lo(uint32_t tmem_d, uint32_t adesc_lo, uint32_t bdesc_lo, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{ .reg .pred p; .reg .b64 da, db; mov.b64 da, {%1, %5}; mov.b64 db, {%2, %5}; setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p; }" ::"r"(tmem_d),
        "r"(adesc_lo), "r"(bdesc_lo), "r"(idesc), "r"(accumulate), "r"(kUmmaDescHiSw128)
        : "memory");
}
__device__ __forceinline__ void umma_f16_lo_pair(uint32_t tmem_d, uint32_t adesc_lo, uint32_t bdesc_lo, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{ .reg .pred p; .reg .b64 da, db; mov.b64 da, {%1, %5}; mov.b64 db, {%2, %5}; setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p; }" ::"r"(tmem_d),
        "r"(adesc_lo), "r"(bdesc_lo), "r"(idesc), "r"(accumulate), "r"(kUmmaDescHiSw128)
        : "memory");
}
// One poll of a barrier phase (the fast path of mbar_wait, for loops that keep their own give-up logic).
__device__ __forceinline__ bool mbar_try(uint32_t bar_addr, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok)
                 : "r"(bar_addr), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ void umma_commit_addr(uint32_t bar_addr)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// The pair's forms: one thread of the leader issues an MMA that spans both CTAs (M 256: 128 rows of A and of the
// accumulator in each CTA, half of B from each), and its commit arrives on the same barrier in both CTAs.
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "h"((uint16_t)3)
                 : "memory");
}


__device__ __forceinline__ void named_bar_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// 32 consecutive accumulator columns of this warp's 32 TMEM lanes: v[j] = D[lane][column + j].
__device__ __forceinline__ void tmem_ld_32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Two runs of 16 consecutive accumulator columns (both loads in flight, then the wait, as one statement so that no
// use of the registers can move ahead of the wait): v[j] = D[lane][c0 + j], w[j] = D[lane][c1 + j].
__device__ __forceinline__ void tmem_ld_16x2(uint32_t taddr0, uint32_t taddr1, uint32_t (&v)[16], uint32_t (&w)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%32];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%33];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(w[0]), "=r"(w[1]), "=r"(w[2]),
          "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]), "=r"(w[8]), "=r"(w[9]), "=r"(w[10]), "=r"(w[11]),
          "=r"(w[12]), "=r"(w[13]), "=r"(w[14]), "=r"(w[15])
        : "r"(taddr0), "r"(taddr1)
        : "memory");
}

// 6-bit (scale, min) of sub-block j from the 12 packed bytes (crates/ferric-gguf/src/lib.rs:795-804); the raw
// block's first 16 bytes sit in `hdr` (x = d | dmin << 16, y..w = the 12 bytes).
__device__ __forceinline__ uint32_t q4k_hdr_byte(const uint4& hdr, int i)
{
    const uint32_t w = i < 4 ? hdr.y : (i < 8 ? hdr.z : hdr.w);
    return (w >> (8 * (i & 3))) & 0xffu;
}
__device__ __forceinline__ void q4k_scale_min(const uint4& hdr, int j, uint32_t& sc, uint32_t& mn)
{
    if (j < 4) {
        sc = q4k_hdr_byte(hdr, j) & 63u;
        mn = q4k_hdr_byte(hdr, j + 4) & 63u;
    } else {
        sc = (q4k_hdr_byte(hdr, j + 4) & 0x0Fu) | ((q4k_hdr_byte(hdr, j - 4) >> 6) << 4);
        mn = (q4k_hdr_byte(hdr, j + 4) >> 4) | ((q4k_hdr_byte(hdr, j) >> 6) << 4);
    }
}
// The same for a sub-block index known only at run time: the 12 bytes as three words, byte i by funnel shift.
__device__ __forceinline__ uint32_t q4k_hdr_byte_dyn(const uint4& hdr, int i)
{
    const uint32_t w = i < 4 ? hdr.y : (i < 8 ? hdr.z : hdr.w);
    return (w >> (8 * (i & 3))) & 0xffu;
}
__device__ __forceinline__ void q4k_scale_min_dyn(const uint4& hdr, int j, uint32_t& sc, uint32_t& mn)
{
    const uint32_t lo_sc = q4k_hdr_byte_dyn(hdr, j & 3), lo_mn = q4k_hdr_byte_dyn(hdr, (j & 3) + 4), hi_b = q4k_hdr_byte_dyn(hdr, (j & 3) + 8);
    if (j < 4) {
        sc = lo_sc & 63u;
        mn = lo_mn & 63u;
    } else {
        sc = (hi_b & 0x0Fu) | ((lo_sc >> 6) << 4);
        mn = (hi_b >> 4) | ((lo_mn >> 6) << 4);
    }
}
}  // namespace ferric
