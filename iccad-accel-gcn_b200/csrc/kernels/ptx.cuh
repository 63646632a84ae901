// Memory-access wrappers used by the SpMM kernels (sm_100a).
#ifndef AGCN_PTX_CUH
#define AGCN_PTX_CUH

namespace agcn {

// dense operand X: read-only path, 16 bytes per lane
__device__ __forceinline__ float4 ld_x4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ float ld_x1(const float *p) { return __ldg(p); }

// sparse operand (col ids / values): streamed once per launch
__device__ __forceinline__ int ld_a(const int *p) { return __ldg(p); }
__device__ __forceinline__ float ld_a(const float *p) { return __ldg(p); }

// result rows
__device__ __forceinline__ void st_y4(float *p, const float4 &v) { *reinterpret_cast<float4 *>(p) = v; }

}  // namespace agcn
#endif
