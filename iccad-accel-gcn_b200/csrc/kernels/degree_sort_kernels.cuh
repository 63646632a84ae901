// Degree sort: stable ascending LSD radix sort of the rows by degree, then the
// CSR permute (and optional symmetric column relabel) that produces the
// degree-ordered `.new_indptr / .new_indices` arrays the Accel-GCN SpMM and
// its partitioner consume (main.cu:62-63, block_level_partition.py:31-38).
//
// One radix pass = per-tile digit histogram -> device-wide exclusive scan of
// the digit-major histogram -> stable scatter.  Stability inside a tile comes
// from ranking keys in tile order: each warp owns a contiguous run of keys and
// ranks 32 consecutive keys at a time with a match-any vote.
#pragma once
#include "primitives.cuh"

namespace agcn {

constexpr int RADIX_BITS = 8;
constexpr int RADIX_BINS = 1 << RADIX_BITS;
constexpr int SORT_BLOCK = 256;
constexpr int SORT_WARPS = SORT_BLOCK / 32;
constexpr int SORT_ITEMS = 16;                       // keys per thread
constexpr int SORT_TILE = SORT_BLOCK * SORT_ITEMS;   // keys per block
constexpr int SORT_WARP_KEYS = 32 * SORT_ITEMS;      // contiguous keys owned by one warp

// degree of every row, the identity permutation, and the maximum degree; four rows per thread with
// 16-byte loads and stores where the caller's row pointers are 16-byte aligned
constexpr int KEYS_ITEMS = 4;

__global__ void __launch_bounds__(256)
degree_keys_kernel(const int *__restrict__ indptr, int64_t n_rows, unsigned *__restrict__ keys,
                   int *__restrict__ rows, int *__restrict__ max_deg, int *__restrict__ err_flag)
{
    const int64_t i0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * KEYS_ITEMS;
    int d_max = 0;
    bool negative = false;
    if (i0 + KEYS_ITEMS <= n_rows && (reinterpret_cast<uintptr_t>(indptr) & 15) == 0) {
        const int4 a = *reinterpret_cast<const int4 *>(indptr + i0);
        const int e = indptr[i0 + KEYS_ITEMS];
        int d[KEYS_ITEMS] = {a.y - a.x, a.z - a.y, a.w - a.z, e - a.w};
#pragma unroll
        for (int k = 0; k < KEYS_ITEMS; k++) {
            if (d[k] < 0) { negative = true; d[k] = 0; }
            d_max = d_max > d[k] ? d_max : d[k];
        }
        *reinterpret_cast<int4 *>(keys + i0) = make_int4(d[0], d[1], d[2], d[3]);      // degrees are >= 0 here
        *reinterpret_cast<int4 *>(rows + i0) = make_int4((int)i0, (int)i0 + 1, (int)i0 + 2, (int)i0 + 3);
    } else {
        for (int64_t i = i0; i < i0 + KEYS_ITEMS && i < n_rows; i++) {
            int d = indptr[i + 1] - indptr[i];
            if (d < 0) { negative = true; d = 0; }
            d_max = d_max > d ? d_max : d;
            keys[i] = (unsigned)d;
            rows[i] = (int)i;
        }
    }
    if (negative) atomicOr(err_flag, 1);
    // one atomic per block, not per warp: at 5e7 rows a million same-address atomics cost more than the pass
    __shared__ int s_max[256 / 32];
    d_max = warp_reduce(d_max, OpMax());
    if (lane_id() == 0) s_max[warp_id()] = d_max;
    __syncthreads();
    if (threadIdx.x == 0) {
        int m = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) m = m > s_max[w] ? m : s_max[w];
        if (m > 0) atomicMax(max_deg, m);
    }
}

// hist[digit * n_tiles + tile] = number of keys of the tile with that digit
__global__ void __launch_bounds__(SORT_BLOCK)
radix_histogram_kernel(const unsigned *__restrict__ keys, int64_t n, int shift, int64_t n_tiles,
                       unsigned *__restrict__ hist)
{
    __shared__ unsigned s_hist[RADIX_BINS];
    for (int b = threadIdx.x; b < RADIX_BINS; b += SORT_BLOCK) s_hist[b] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * SORT_TILE;
#pragma unroll
    for (int k = 0; k < SORT_ITEMS; k++) {
        const int64_t i = base + (int64_t)k * SORT_BLOCK + threadIdx.x;
        if (i < n) atomicAdd(&s_hist[(keys[i] >> shift) & (RADIX_BINS - 1)], 1u);
    }
    __syncthreads();
    for (int b = threadIdx.x; b < RADIX_BINS; b += SORT_BLOCK)
        hist[(int64_t)b * n_tiles + blockIdx.x] = s_hist[b];
}

// Stable scatter of one tile.  hist_scanned is the exclusive scan of `hist`.
__global__ void __launch_bounds__(SORT_BLOCK)
radix_scatter_kernel(const unsigned *__restrict__ keys_in, const int *__restrict__ vals_in, int64_t n, int shift,
                     int64_t n_tiles, const unsigned *__restrict__ hist_scanned,
                     unsigned *__restrict__ keys_out, int *__restrict__ vals_out)
{
    __shared__ unsigned s_count[SORT_WARPS][RADIX_BINS];   // keys of each digit seen by each warp
    __shared__ unsigned s_base[RADIX_BINS];                // global position of the tile's first key of a digit
    for (int b = threadIdx.x; b < SORT_WARPS * RADIX_BINS; b += SORT_BLOCK) (&s_count[0][0])[b] = 0;
    __syncthreads();

    const int w = warp_id(), lane = lane_id();
    const int64_t warp_base = (int64_t)blockIdx.x * SORT_TILE + (int64_t)w * SORT_WARP_KEYS;
    unsigned key[SORT_ITEMS];
    int val[SORT_ITEMS];
    unsigned rank[SORT_ITEMS];   // position of the key among the warp's keys of the same digit
#pragma unroll
    for (int k = 0; k < SORT_ITEMS; k++) {
        const int64_t i = warp_base + k * 32 + lane;
        const bool live = i < n;
        key[k] = live ? keys_in[i] : 0xffffffffu;
        val[k] = live ? vals_in[i] : 0;
        // dead keys vote in a bin of their own (digit id RADIX_BINS) and are never written
        const unsigned digit = live ? ((key[k] >> shift) & (RADIX_BINS - 1)) : (unsigned)RADIX_BINS;
        const unsigned peers = __match_any_sync(FULL_MASK, digit);
        const unsigned before = __popc(peers & ((1u << lane) - 1u));
        unsigned seen = 0;
        if (live) seen = s_count[w][digit];
        __syncwarp();
        if (live && before == 0) s_count[w][digit] = seen + __popc(peers);
        __syncwarp();
        rank[k] = seen + before;
    }
    __syncthreads();
    // digit d: exclusive prefix over the warps, plus the tile's global base
    for (int d = threadIdx.x; d < RADIX_BINS; d += SORT_BLOCK) {
        unsigned run = 0;
        for (int ww = 0; ww < SORT_WARPS; ww++) {
            const unsigned c = s_count[ww][d];
            s_count[ww][d] = run;
            run += c;
        }
        s_base[d] = hist_scanned[(int64_t)d * n_tiles + blockIdx.x];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SORT_ITEMS; k++) {
        const int64_t i = warp_base + k * 32 + lane;
        if (i < n) {
            const unsigned digit = (key[k] >> shift) & (RADIX_BINS - 1);
            const int64_t pos = (int64_t)s_base[digit] + s_count[w][digit] + rank[k];
            keys_out[pos] = key[k];
            vals_out[pos] = val[k];
        }
    }
}

// inverse permutation: new_id[perm[r]] = r
__global__ void __launch_bounds__(256)
invert_perm_kernel(const int *__restrict__ perm, int64_t n, int *__restrict__ new_id)
{
    const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n) new_id[perm[r]] = (int)r;
}

// CSR permute.  Each block produces PERMUTE_TILE consecutive output nonzeros:
// it finds the (non-empty) output rows its range touches, stages their new and
// old row starts in shared memory, and every thread locates the row of each of
// its nonzeros by binary search there.  new_id == nullptr keeps column ids.
constexpr int PERMUTE_BLOCK = 256;
constexpr int PERMUTE_ITEMS = 8;
constexpr int PERMUTE_TILE = PERMUTE_BLOCK * PERMUTE_ITEMS;

__device__ __forceinline__ int64_t upper_bound_i32(const int *a, int64_t lo, int64_t hi, int64_t key)
{
    // first index in [lo, hi) with a[index] > key
    while (lo < hi) {
        const int64_t mid = lo + ((hi - lo) >> 1);
        if ((int64_t)a[mid] <= key) lo = mid + 1; else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(PERMUTE_BLOCK)
csr_permute_kernel(const int *__restrict__ old_indptr, const int *__restrict__ old_indices,
                   const float *__restrict__ old_vals, const int *__restrict__ perm,
                   const int *__restrict__ new_indptr, const int *__restrict__ new_id,
                   int64_t n_rows, int64_t nnz, int *__restrict__ new_indices, float *__restrict__ new_vals,
                   int *__restrict__ err_flag)
{
    __shared__ int s_new_start[PERMUTE_TILE + 2];
    __shared__ int s_old_start[PERMUTE_TILE + 2];
    __shared__ int64_t s_rows[2];
    const int64_t p0 = (int64_t)blockIdx.x * PERMUTE_TILE;
    const int64_t p1 = p0 + PERMUTE_TILE < nnz ? p0 + PERMUTE_TILE : nnz;
    const int ip0 = old_indptr[0];
    if (threadIdx.x == 0) {
        // rows r_lo..r_hi own the nonzeros p0..p1-1: r = last row with new_indptr[r] <= p
        s_rows[0] = upper_bound_i32(new_indptr, 0, n_rows + 1, p0) - 1;
        s_rows[1] = upper_bound_i32(new_indptr, 0, n_rows + 1, p1 - 1) - 1;
    }
    __syncthreads();
    const int64_t r_lo = s_rows[0], r_hi = s_rows[1];
    const int n_span = (int)(r_hi - r_lo + 1);    // <= PERMUTE_TILE: every row in the span is non-empty
    for (int k = threadIdx.x; k <= n_span; k += PERMUTE_BLOCK) {
        s_new_start[k] = new_indptr[r_lo + k];
        if (k < n_span) s_old_start[k] = old_indptr[perm[r_lo + k]] - ip0;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < PERMUTE_ITEMS; k++) {
        const int64_t p = p0 + (int64_t)k * PERMUTE_BLOCK + threadIdx.x;
        if (p < p1) {
            const int rr = (int)upper_bound_i32(s_new_start, 0, n_span, p) - 1;
            const int64_t src = (int64_t)s_old_start[rr] + (p - s_new_start[rr]);
            int c = old_indices[src];
            if (new_id != nullptr) {
                if (c < 0 || c >= n_rows) { atomicOr(err_flag, 1); c = 0; }
                c = new_id[c];
            }
            new_indices[p] = c;
            if (new_vals != nullptr) new_vals[p] = old_vals[src];
        }
    }
}

}  // namespace agcn
