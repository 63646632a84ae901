// Block-level partitioner: degree-ordered CSR row pointers -> `.block4`
// metadata, bit-exact with the sequential walk of the reference script
// (block_level_partition.py:48-103) for ANY degree sequence, sorted or not.
//
// The walk is a state machine over rows, but its output has a closed form per
// row once the start of the row's run of equal consecutive degrees is known:
//   degree 0            -> no tuple
//   1 <= D <= 384       -> the row opens a tuple iff (row - run_start) % R(D) == 0;
//                          the tuple covers j = min(R(D), rows left in the run) rows
//   D > 384             -> ceil(D / 384) tuples of <= 384 nonzeros each
// with R(D), w(D) the pattern tables of block_level_partition.py:7-21 and the
// fall-backs of :56-63.  So: (A) a max-scan finds run starts, (B) a sum-scan
// of per-row tuple counts finds output offsets, (C) every row writes its own
// tuples.  Each phase works on tiles of PART_TILE rows staged through shared
// memory; the two cross-tile scans are single-block kernels.
#pragma once
#include "primitives.cuh"

namespace agcn {

constexpr int PART_DEG_BOUND = 384;   // 12 warps x 32 nonzeros: a format constant of .block4
constexpr int PART_BLOCK = 256;
constexpr int PART_ITEMS = 8;
constexpr int PART_TILE = PART_BLOCK * PART_ITEMS;
constexpr int PART_MAX_ROWS_PER_TUPLE = 12;
constexpr int PART_HALO = PART_MAX_ROWS_PER_TUPLE + 1;   // rows looked at past a tile

// rows per tuple R(D) and nonzeros per virtual warp w(D), 1 <= D <= 384
__device__ __forceinline__ int part_rows_per_tuple(int d)
{
    return d <= 32 ? 12 : d <= 64 ? 6 : d <= 96 ? 4 : d <= 128 ? 3 : d <= 191 ? 2 : 1;
}
__device__ __forceinline__ int part_warp_nz(int d)
{
    if (d >= 192) return 32;
    const int f = 12 / part_rows_per_tuple(d);
    return (d + f - 1) / f;
}

// Shared-memory view of indptr[tile_first - 1 .. tile_first + PART_TILE + PART_HALO]
// (indices clamped to [0, n_rows]); deg(i) is valid for tile_first-1 <= i and
// i < tile_first + PART_TILE + PART_HALO, and returns -1 for rows that do not exist.
// Every thread walks PART_ITEMS consecutive rows, so the threads of a warp read words PART_ITEMS
// apart: one pad word per 32 keeps those reads on different banks (unpadded they collide 8 ways).
__device__ __forceinline__ int part_pad(int k) { return k + (k >> 5); }

struct PartTile {
    int *s_ip;
    int64_t first;    // first row of the tile
    int64_t n_rows;
    __device__ __forceinline__ int ip(int64_t i) const { return s_ip[part_pad((int)(i - first + 1))]; }
    __device__ __forceinline__ int deg(int64_t i) const
    {
        if (i < 0 || i >= n_rows) return -1;
        return ip(i + 1) - ip(i);
    }
};

constexpr int PART_TILE_INTS = PART_TILE + PART_HALO + 2;                  // row pointers a tile looks at
constexpr int PART_SMEM_INTS = PART_TILE_INTS + PART_TILE_INTS / 32 + 1;   // the same, padded

__device__ __forceinline__ PartTile part_load_tile(const int *__restrict__ indptr, int64_t n_rows, int *s_ip)
{
    PartTile t;
    t.s_ip = s_ip;
    t.first = (int64_t)blockIdx.x * PART_TILE;
    t.n_rows = n_rows;
    for (int k = threadIdx.x; k < PART_TILE_INTS; k += PART_BLOCK) {
        int64_t i = t.first - 1 + k;
        i = i < 0 ? 0 : (i > n_rows ? n_rows : i);
        s_ip[part_pad(k)] = indptr[i];
    }
    __syncthreads();
    return t;
}

// (A) per tile: index of the last row in the tile that starts a run (-1 if none)
__global__ void __launch_bounds__(PART_BLOCK)
part_run_heads_kernel(const int *__restrict__ indptr, int64_t n_rows, int *__restrict__ tile_last_head,
                      int *__restrict__ err_flag)
{
    __shared__ int s_ip[PART_SMEM_INTS];
    __shared__ int s_warp[PART_BLOCK / 32];
    const PartTile t = part_load_tile(indptr, n_rows, s_ip);
    int last = -1;
    bool negative = false;
#pragma unroll
    for (int k = 0; k < PART_ITEMS; k++) {
        const int64_t i = t.first + (int64_t)threadIdx.x * PART_ITEMS + k;
        if (i < n_rows) {
            const int d = t.deg(i);
            negative |= d < 0;
            if (i == 0 || d != t.deg(i - 1)) last = (int)i;
        }
    }
    if (negative) atomicOr(err_flag, 1);
    last = warp_reduce(last, OpMax());
    if (lane_id() == 0) s_warp[warp_id()] = last;
    __syncthreads();
    if (threadIdx.x == 0) {
        int m = -1;
        for (int w = 0; w < PART_BLOCK / 32; w++) m = m > s_warp[w] ? m : s_warp[w];
        tile_last_head[blockIdx.x] = m;
    }
}

// Number of tuples each of this thread's PART_ITEMS rows opens.
// incoming_head = start of the run that is open when the tile begins.
__device__ __forceinline__ void part_row_counts(const PartTile &t, int incoming_head, int *s_scan,
                                                int (&cnt)[PART_ITEMS])
{
    const int64_t my_first = t.first + (int64_t)threadIdx.x * PART_ITEMS;
    // last run head among this thread's rows, then an exclusive max-scan over the block
    int head_local = -1;
#pragma unroll
    for (int k = 0; k < PART_ITEMS; k++) {
        const int64_t i = my_first + k;
        if (i < t.n_rows && (i == 0 || t.deg(i) != t.deg(i - 1))) head_local = (int)i;
    }
    int unused_total;
    int run_head = block_scan_exclusive<PART_BLOCK>(head_local, OpMax(), -1, unused_total, s_scan);
    run_head = run_head > incoming_head ? run_head : incoming_head;
#pragma unroll
    for (int k = 0; k < PART_ITEMS; k++) {
        const int64_t i = my_first + k;
        int c = 0;
        if (i < t.n_rows) {
            const int d = t.deg(i);
            if (i == 0 || d != t.deg(i - 1)) run_head = (int)i;
            if (d > PART_DEG_BOUND) c = (d + PART_DEG_BOUND - 1) / PART_DEG_BOUND;
            else if (d >= 1) c = ((int)i - run_head) % part_rows_per_tuple(d) == 0 ? 1 : 0;
        }
        cnt[k] = c;
    }
}

// (B) per tile: number of tuples the tile's rows open
__global__ void __launch_bounds__(PART_BLOCK)
part_count_kernel(const int *__restrict__ indptr, int64_t n_rows, const int *__restrict__ tile_incoming_head,
                  int64_t *__restrict__ tile_count)
{
    __shared__ int s_ip[PART_SMEM_INTS];
    __shared__ int s_scan[PART_BLOCK / 32 + 1];
    __shared__ int64_t s_sum[PART_BLOCK / 32];
    const PartTile t = part_load_tile(indptr, n_rows, s_ip);
    int cnt[PART_ITEMS];
    part_row_counts(t, tile_incoming_head[blockIdx.x], s_scan, cnt);
    int64_t sum = 0;
#pragma unroll
    for (int k = 0; k < PART_ITEMS; k++) sum += cnt[k];
    sum = warp_reduce(sum, OpAdd());
    if (lane_id() == 0) s_sum[warp_id()] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        int64_t s = 0;
        for (int w = 0; w < PART_BLOCK / 32; w++) s += s_sum[w];
        tile_count[blockIdx.x] = s;
    }
}

// (C) every row that opens tuples writes them at its scanned offset.  A row of degree D > 384 owns
// ceil(D / 384) tuples -- thousands for a hub row -- so rows with more than PART_INLINE_TUPLES are
// queued in shared memory and written by the whole block together instead of by their one thread.
constexpr int PART_INLINE_TUPLES = 8;
constexpr int PART_HEAVY_QUEUE = 128;

__global__ void __launch_bounds__(PART_BLOCK)
part_emit_kernel(const int *__restrict__ indptr, int64_t n_rows, const int *__restrict__ tile_incoming_head,
                 const int64_t *__restrict__ tile_offset, int4 *__restrict__ block4)
{
    __shared__ int s_ip[PART_SMEM_INTS];
    __shared__ int s_scan[PART_BLOCK / 32 + 1];
    __shared__ int s_heavy_n;
    __shared__ int s_heavy_row[PART_HEAVY_QUEUE], s_heavy_deg[PART_HEAVY_QUEUE], s_heavy_loc[PART_HEAVY_QUEUE];
    __shared__ int64_t s_heavy_out[PART_HEAVY_QUEUE];
    if (threadIdx.x == 0) s_heavy_n = 0;
    const PartTile t = part_load_tile(indptr, n_rows, s_ip);      // synchronises the block
    int cnt[PART_ITEMS];
    part_row_counts(t, tile_incoming_head[blockIdx.x], s_scan, cnt);
    int sum = 0;
#pragma unroll
    for (int k = 0; k < PART_ITEMS; k++) sum += cnt[k];
    int tile_total;
    const int ex = block_scan_exclusive<PART_BLOCK>(sum, OpAdd(), 0, tile_total, s_scan);
    int64_t out = tile_offset[blockIdx.x] + ex;
    const int ip0 = indptr[0];
    const int64_t my_first = t.first + (int64_t)threadIdx.x * PART_ITEMS;
#pragma unroll
    for (int k = 0; k < PART_ITEMS; k++) {
        if (cnt[k] == 0) continue;
        const int64_t i = my_first + k;
        const int d = t.deg(i);
        const int loc = t.ip(i) - ip0;
        if (d <= PART_DEG_BOUND) {
            const int rows_max = part_rows_per_tuple(d);
            int j = 1;
            while (j < rows_max && t.deg(i + j) == d) j++;
            block4[out] = make_int4(d, (int)i, loc, (part_warp_nz(d) << 16) + j);
            out += 1;
        } else {
            int slot = PART_HEAVY_QUEUE;
            if (cnt[k] > PART_INLINE_TUPLES) slot = atomicAdd(&s_heavy_n, 1);
            if (slot < PART_HEAVY_QUEUE) {
                s_heavy_row[slot] = (int)i; s_heavy_deg[slot] = d; s_heavy_loc[slot] = loc; s_heavy_out[slot] = out;
            } else {
                for (int c = 0; c < cnt[k]; c++) {
                    const int done = c * PART_DEG_BOUND;
                    const int take = d - done < PART_DEG_BOUND ? d - done : PART_DEG_BOUND;
                    block4[out + c] = make_int4(d, (int)i, loc + done, take);
                }
            }
            out += cnt[k];
        }
    }
    __syncthreads();
    const int n_heavy = s_heavy_n < PART_HEAVY_QUEUE ? s_heavy_n : PART_HEAVY_QUEUE;
    for (int q = 0; q < n_heavy; q++) {
        const int d = s_heavy_deg[q], row = s_heavy_row[q], loc = s_heavy_loc[q];
        const int64_t o = s_heavy_out[q];
        const int n_tuples = (d + PART_DEG_BOUND - 1) / PART_DEG_BOUND;
        for (int c = threadIdx.x; c < n_tuples; c += PART_BLOCK) {
            const int done = c * PART_DEG_BOUND;
            const int take = d - done < PART_DEG_BOUND ? d - done : PART_DEG_BOUND;
            block4[o + c] = make_int4(d, row, loc + done, take);
        }
    }
}

}  // namespace agcn
