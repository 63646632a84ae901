// Host-side helpers shared by the C-ABI translation units: error reporting,
// checked CUDA calls, scratch buffers and the device-wide prefix sum.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <cstdarg>
#include <cstdio>
#include <vector>

#include "../../include/accelgcn.h"

namespace agcn {

void set_error(const char *fmt, ...);
void clear_error();

#define AGCN_CUDA(call)                                                                          \
    do {                                                                                         \
        cudaError_t agcn_e_ = (call);                                                            \
        if (agcn_e_ != cudaSuccess) {                                                            \
            ::agcn::set_error("%s: %s (%s:%d)", #call, cudaGetErrorString(agcn_e_), __FILE__, __LINE__); \
            return AGCN_ERR_CUDA;                                                                \
        }                                                                                        \
    } while (0)

// kernel launch: `kernel` is a function name or a pointer to an instantiated template
#ifndef AGCN_KERNEL
#define AGCN_KERNEL(kernel, grid, block, stream, ...) kernel<<<(grid), (block), 0, (stream)>>>(__VA_ARGS__)
#endif

#define AGCN_LAUNCH_CHECK(name)                                                                  \
    do {                                                                                         \
        cudaError_t agcn_e_ = cudaGetLastError();                                                \
        if (agcn_e_ != cudaSuccess) {                                                            \
            ::agcn::set_error("launch of %s: %s (%s:%d)", name, cudaGetErrorString(agcn_e_), __FILE__, __LINE__); \
            return AGCN_ERR_CUDA;                                                                \
        }                                                                                        \
    } while (0)

#define AGCN_REQUIRE(cond, ...)                                                                  \
    do {                                                                                         \
        if (!(cond)) { ::agcn::set_error(__VA_ARGS__); return AGCN_ERR_INVALID; }                \
    } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Device allocations that free themselves when the call returns.
class DeviceScratch {
public:
    DeviceScratch() = default;
    DeviceScratch(const DeviceScratch &) = delete;
    DeviceScratch &operator=(const DeviceScratch &) = delete;
    ~DeviceScratch() { for (void *p : ptrs_) cudaFree(p); }
    // returns nullptr (and records the error) on failure
    template <typename T> T *alloc(int64_t count)
    {
        void *p = nullptr;
        const size_t bytes = (size_t)(count > 0 ? count : 1) * sizeof(T);
        cudaError_t e = cudaMalloc(&p, bytes);
        if (e != cudaSuccess) {
            set_error("cudaMalloc(%zu bytes): %s", bytes, cudaGetErrorString(e));
            return nullptr;
        }
        ptrs_.push_back(p);
        return static_cast<T *>(p);
    }
private:
    std::vector<void *> ptrs_;
};

#define AGCN_ALLOC(var, scratch, type, count)                  \
    type *var = (scratch).alloc<type>(count);                  \
    if (var == nullptr) return AGCN_ERR_CUDA

// Exclusive prefix sums used by several entry points (defined in scan.cu).
// tile_sums must hold ceil(n / 2048) elements.  total_out may be null.
int exclusive_scan_i32_i64(const int *in, int64_t *out, int64_t n, int64_t *tile_sums, int64_t *total_out, cudaStream_t s);
int exclusive_scan_u32_u32(const unsigned *in, unsigned *out, int64_t n, unsigned *tile_sums, cudaStream_t s);
int exclusive_scan_u32_i32(const unsigned *in, int *out, int64_t n, int *tile_sums, cudaStream_t s);
int64_t scan_tiles(int64_t n);

}  // namespace agcn
