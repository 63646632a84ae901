// Warp- and block-level building blocks shared by the preprocessing kernels
// (degree sort, prefix sums, block-meta emission).  Device code only.
#pragma once
#include <stdint.h>

namespace agcn {

constexpr unsigned FULL_MASK = 0xffffffffu;

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }

struct OpAdd {
    template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a + b; }
};
struct OpMax {
    template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a > b ? a : b; }
};

// Inclusive scan across the 32 lanes of a warp.
template <typename T, typename Op>
__device__ __forceinline__ T warp_scan_inclusive(T v, Op op)
{
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        T t = __shfl_up_sync(FULL_MASK, v, d);
        if (lane_id() >= d) v = op(t, v);
    }
    return v;
}

template <typename T, typename Op>
__device__ __forceinline__ T warp_reduce(T v, Op op)
{
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = op(v, __shfl_xor_sync(FULL_MASK, v, d));
    return v;
}

// Exclusive scan of one value per thread over a block of BLOCK threads
// (BLOCK a multiple of 32, at most 1024).  `identity` is the neutral element
// of `op`.  `total` receives the reduction over the block.  `s_warp` is a
// shared array of BLOCK/32 + 1 elements; the call synchronises the block.
template <int BLOCK, typename T, typename Op>
__device__ __forceinline__ T block_scan_exclusive(T v, Op op, T identity, T &total, T *s_warp)
{
    constexpr int NW = BLOCK / 32;
    const T incl = warp_scan_inclusive(v, op);
    if (lane_id() == 31) s_warp[warp_id()] = incl;
    __syncthreads();
    if (warp_id() == 0) {
        T w = lane_id() < NW ? s_warp[lane_id()] : identity;
        const T wi = warp_scan_inclusive(w, op);
        // exclusive prefix of the warp totals
        T we = __shfl_up_sync(FULL_MASK, wi, 1);
        if (lane_id() == 0) we = identity;
        if (lane_id() < NW) s_warp[lane_id()] = we;
        if (lane_id() == NW - 1) s_warp[NW] = wi;
    }
    __syncthreads();
    T excl = __shfl_up_sync(FULL_MASK, incl, 1);
    if (lane_id() == 0) excl = identity;
    const T res = op(s_warp[warp_id()], excl);
    total = s_warp[NW];
    __syncthreads();   // s_warp may be reused by the caller
    return res;
}

// ---------------------------------------------------------------------------
// Device-wide exclusive prefix sum: reduce tiles -> scan tile sums (one
// block) -> scan tiles with their offsets.  TIn is the element type read,
// TAcc the type accumulated and written.
// ---------------------------------------------------------------------------
constexpr int SCAN_BLOCK = 256;
constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_TILE = SCAN_BLOCK * SCAN_ITEMS;

template <typename TIn, typename TAcc>
__global__ void __launch_bounds__(SCAN_BLOCK)
scan_tile_reduce_kernel(const TIn *__restrict__ in, int64_t n, TAcc *__restrict__ tile_sum)
{
    __shared__ TAcc s_warp[SCAN_BLOCK / 32];
    const int64_t base = (int64_t)blockIdx.x * SCAN_TILE;
    TAcc acc = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        const int64_t i = base + (int64_t)k * SCAN_BLOCK + threadIdx.x;
        if (i < n) acc += (TAcc)in[i];
    }
    acc = warp_reduce(acc, OpAdd());
    if (lane_id() == 0) s_warp[warp_id()] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        TAcc t = 0;
        for (int w = 0; w < SCAN_BLOCK / 32; w++) t += s_warp[w];
        tile_sum[blockIdx.x] = t;
    }
}

// One block scans an array of any length in place (exclusive), carrying the
// running value from chunk to chunk.  total_out (may be null) gets the sum.
template <typename T, typename Op>
__global__ void __launch_bounds__(1024)
single_block_scan_exclusive_kernel(T *__restrict__ data, int64_t n, T identity, T *__restrict__ total_out)
{
    __shared__ T s_warp[1024 / 32 + 1];
    Op op;
    T carry = identity;
    for (int64_t base = 0; base < n; base += 1024) {
        const int64_t i = base + threadIdx.x;
        const T v = i < n ? data[i] : identity;
        T total;
        const T ex = block_scan_exclusive<1024>(v, op, identity, total, s_warp);
        if (i < n) data[i] = op(carry, ex);
        carry = op(carry, total);
    }
    if (total_out != nullptr && threadIdx.x == 0) *total_out = carry;
}

template <typename TIn, typename TAcc, typename TOut>
__global__ void __launch_bounds__(SCAN_BLOCK)
scan_tile_downsweep_kernel(const TIn *__restrict__ in, int64_t n, const TAcc *__restrict__ tile_offset,
                           TOut *__restrict__ out)
{
    // blocked arrangement through shared memory so that both the loads and
    // the stores are coalesced
    __shared__ TAcc s_vals[SCAN_TILE];
    __shared__ TAcc s_warp[SCAN_BLOCK / 32 + 1];
    const int64_t base = (int64_t)blockIdx.x * SCAN_TILE;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        const int j = k * SCAN_BLOCK + threadIdx.x;
        const int64_t i = base + j;
        s_vals[j] = i < n ? (TAcc)in[i] : (TAcc)0;
    }
    __syncthreads();
    TAcc local[SCAN_ITEMS];
    TAcc sum = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        local[k] = sum;
        sum += s_vals[threadIdx.x * SCAN_ITEMS + k];
    }
    TAcc total;
    const TAcc ex = block_scan_exclusive<SCAN_BLOCK>(sum, OpAdd(), (TAcc)0, total, s_warp);
    const TAcc off = tile_offset[blockIdx.x];
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) s_vals[threadIdx.x * SCAN_ITEMS + k] = off + ex + local[k];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        const int j = k * SCAN_BLOCK + threadIdx.x;
        const int64_t i = base + j;
        if (i < n) out[i] = (TOut)s_vals[j];
    }
}

}  // namespace agcn
