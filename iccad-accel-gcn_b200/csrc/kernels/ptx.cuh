// Memory-access wrappers of the SpMM kernels (sm_100a inline PTX).
//
// The gather is bound by what L2 can deliver, so what stays in L2 matters:
//  - the dense operand X is re-read once per nonzero of its column and should
//    stay resident: loads carry an L2 evict_last policy;
//  - the sparse operand (column ids, values) and the .block4 tuples are read
//    exactly once per launch: loads bypass L1 allocation and carry an L2
//    evict_first policy, so that streaming 8 bytes per nonzero does not push X
//    rows out of L2;
//  - result rows are written once and not read again by the kernel: stores
//    carry evict_first as well.
#ifndef AGCN_PTX_CUH
#define AGCN_PTX_CUH
#include <stdint.h>

namespace agcn {

struct L2Policies {
    uint64_t keep;     // evict_last
    uint64_t stream;   // evict_first
};

__device__ __forceinline__ L2Policies make_l2_policies()
{
    L2Policies p;
    asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p.keep));
    asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p.stream));
    return p;
}

// dense operand X: read-only path, 16 bytes per lane, keep in L2
__device__ __forceinline__ float4 ld_x4(const float *p, uint64_t policy)
{
    float4 v;
    asm("ld.global.nc.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p), "l"(policy));
    return v;
}
__device__ __forceinline__ float ld_x1(const float *p, uint64_t policy)
{
    float v;
    asm("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(policy));
    return v;
}

// sparse operand (col ids / values): streamed once per launch
__device__ __forceinline__ int ld_a(const int *p, uint64_t policy)
{
    int v;
    asm("ld.global.nc.L1::no_allocate.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(policy));
    return v;
}
__device__ __forceinline__ float ld_a(const float *p, uint64_t policy)
{
    float v;
    asm("ld.global.nc.L1::no_allocate.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(policy));
    return v;
}

// result rows: written once
__device__ __forceinline__ void st_y4(float *p, const float4 &v, uint64_t policy)
{
    asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;"
                 :: "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "l"(policy) : "memory");
}
__device__ __forceinline__ void st_y1(float *p, float v, uint64_t policy)
{
    asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;" :: "l"(p), "f"(v), "l"(policy) : "memory");
}

}  // namespace agcn
#endif
