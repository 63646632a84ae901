// Column tiling of A for the gather SpMM (no counterpart in the reference, whose kernel gathers
// X rows un-tiled, spmm_accel.cu:55-78).
//
// The SpMM re-reads a row of X once per nonzero of that column, so it runs at L2 speed only while
// the rows it touches stay L2-resident.  When X is larger than that, A's columns are cut into
// ranges whose slab of X fits, and the nonzeros are regrouped range by range: the product then
// runs one range after the other (the first stores Y, the later ones add to it, in a fixed order),
// every launch touches one slab of X only, and A is still streamed exactly once in total.
//
// Layout produced here ("range-major CSR"): the nonzeros of range 0 of every row, in row order and
// in their original order inside a row, then those of range 1, and so on; one row-pointer array
// per range.  Each range is then an ordinary CSR matrix over all rows, and gets its own `.block4`
// metadata from the ordinary partitioner -- the format is untouched.
#pragma once
#include "primitives.cuh"

namespace agcn {

constexpr int TILE_MAX_RANGES = 32;      // one lane of a warp keeps the running position of one range
constexpr int TILE_WARPS = 8;            // rows per thread block (one warp per row)

struct TileBounds {
    int n_ranges;
    int bound[TILE_MAX_RANGES + 1];      // range k = columns [bound[k], bound[k+1])
};

__device__ __forceinline__ int tile_range_of(const TileBounds &b, int col)
{
    int k = 0;
    while (k + 1 < b.n_ranges && col >= b.bound[k + 1]) k++;
    return k;
}

// count[k * (n_rows + 1) + row] = nonzeros of `row` whose column lies in range k; entry n_rows of
// every range is written as 0, so that an exclusive scan of the whole array gives every
// (range, row) segment its position in the range-major order.
__global__ void __launch_bounds__(TILE_WARPS * 32)
tile_count_kernel(const int *__restrict__ indptr, const int *__restrict__ idx, int64_t n_rows, const TileBounds b,
                  int *__restrict__ count)
{
    const int64_t row = (int64_t)blockIdx.x * TILE_WARPS + warp_id();
    if (row > n_rows) return;
    const int lane = lane_id();
    int mine = 0;                         // lane k: nonzeros of this row in range k
    if (row < n_rows) {
        const int p0 = indptr[row], p1 = indptr[row + 1];
        for (int p = p0 + lane; p - lane < p1; p += 32) {
            const bool live = p < p1;
            const int key = live ? tile_range_of(b, idx[p]) : -1;
            for (int k = 0; k < b.n_ranges; k++) {
                const unsigned votes = __ballot_sync(FULL_MASK, key == k);
                if (lane == k) mine += __popc(votes);
            }
        }
    }
    if (lane < b.n_ranges) count[(int64_t)lane * (n_rows + 1) + row] = mine;
}

// Moves every nonzero to its place: position[k * (n_rows + 1) + row] is where the (range k, row)
// segment starts.  Inside a segment the nonzeros keep their original order (ranked with a
// match-any vote, 32 at a time).
__global__ void __launch_bounds__(TILE_WARPS * 32)
tile_place_kernel(const int *__restrict__ indptr, const int *__restrict__ idx, const float *__restrict__ val,
                  int64_t n_rows, const TileBounds b, const int64_t *__restrict__ position,
                  int *__restrict__ idx_out, float *__restrict__ val_out)
{
    const int64_t row = (int64_t)blockIdx.x * TILE_WARPS + warp_id();
    if (row >= n_rows) return;
    const int lane = lane_id();
    int64_t next = lane < b.n_ranges ? position[(int64_t)lane * (n_rows + 1) + row] : 0;   // lane k: next free slot of range k
    const int p0 = indptr[row], p1 = indptr[row + 1];
    for (int p = p0 + lane; p - lane < p1; p += 32) {
        const bool live = p < p1;
        const int key = live ? tile_range_of(b, idx[p]) : TILE_MAX_RANGES;      // dead lanes vote in a bin of their own
        const unsigned peers = __match_any_sync(FULL_MASK, key);
        const int before = __popc(peers & ((1u << lane) - 1u));
        const int64_t base = __shfl_sync(FULL_MASK, next, key & 31);
        if (live) {
            idx_out[base + before] = idx[p];
            val_out[base + before] = val[p];
        }
        for (int k = 0; k < b.n_ranges; k++) {
            const unsigned votes = __ballot_sync(FULL_MASK, key == k);
            if (lane == k) next += __popc(votes);
        }
    }
}

// Row pointers of every range, relative to the range's first nonzero (int32, like any indptr).
__global__ void __launch_bounds__(256)
tile_indptr_kernel(const int64_t *__restrict__ position, int64_t n_rows, int n_ranges, int *__restrict__ indptr_out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t per = n_rows + 1;
    if (i >= per * n_ranges) return;
    const int64_t k = i / per;
    indptr_out[i] = (int)(position[i] - position[k * per]);
}

}  // namespace agcn
