// The (value, exchange number) pair stores and loads of the two-step pushed all-reduce (kernels_tpwide.cu), shared with
// the product kernels that scatter their result themselves.
#pragma once
#include <stdint.h>

namespace ferric {

__device__ __forceinline__ unsigned wide_stamp(const unsigned* epoch)
{
    unsigned e;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(e) : "l"(epoch));
    return e + 1;
}
__device__ __forceinline__ void store_pairs4(uint2* dst, float4 v, unsigned stamp)
{
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(__float_as_uint(v.x)), "r"(stamp),
                 "r"(__float_as_uint(v.y)), "r"(stamp) : "memory");
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 2), "r"(__float_as_uint(v.z)), "r"(stamp),
                 "r"(__float_as_uint(v.w)), "r"(stamp) : "memory");
}
__device__ __forceinline__ void load_pairs4(const uint2* src, uint4& a, uint4& b)
{
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(src));
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(src + 2));
}

}  // namespace ferric
