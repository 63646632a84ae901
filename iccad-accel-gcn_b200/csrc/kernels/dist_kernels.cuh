// Kernels that cut one rank's block out of the degree-ordered matrix for the row-sharded SpMM
// (two row ranges per rank, see layout.cu) and rename column ids to positions in the gathered
// dense operand.  The reference is single-GPU and has no counterpart.
#pragma once
#include "primitives.cuh"

namespace agcn {

constexpr int DIST_MAX_WORLD = 64;

// Row ranges of every rank (int32: row ids fit the .block4 format) and the shape of the gathered
// operand: world blocks of `per` rows, exchanged in `chunks` slices of per / chunks rows each.
// Position of local row j of rank g in the gathered operand:
//     slice c = j / rows_per_chunk,  i = j % rows_per_chunk  ->  c * (world * rows_per_chunk) + g * rows_per_chunk + i
// (with one chunk this is simply g * per + j).
struct DistLayout {
    int world, chunks;
    int per, rows_per_chunk;
    int light0[DIST_MAX_WORLD], light1[DIST_MAX_WORLD];     // rank g: rows [light0, light1) ...
    int heavy0[DIST_MAX_WORLD], heavy1[DIST_MAX_WORLD];     // ... then rows [heavy0, heavy1)
};

__host__ __device__ __forceinline__ int dist_position(const DistLayout &L, int g, int j)
{
    const int c = j / L.rows_per_chunk, i = j - c * L.rows_per_chunk;
    return c * (L.world * L.rows_per_chunk) + g * L.rows_per_chunk + i;
}

// position in the gathered operand of row r of the degree-ordered matrix
__host__ __device__ __forceinline__ int dist_new_id(const DistLayout &L, int r)
{
    for (int g = 0; g < L.world; g++) {
        if (r >= L.light0[g] && r < L.light1[g]) return dist_position(L, g, r - L.light0[g]);
        if (r >= L.heavy0[g] && r < L.heavy1[g]) return dist_position(L, g, (L.light1[g] - L.light0[g]) + (r - L.heavy0[g]));
    }
    return -1;
}

// Row pointers of rank g's block: its light rows, its heavy rows, then empty padding rows up to `per`.
__global__ void __launch_bounds__(256)
dist_local_indptr_kernel(const int *__restrict__ indptr, const DistLayout L, int g, int *__restrict__ out)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j > L.per) return;
    const int n_light = L.light1[g] - L.light0[g], n_heavy = L.heavy1[g] - L.heavy0[g];
    const int light_nz = indptr[L.light1[g]] - indptr[L.light0[g]];
    int v;
    if (j <= n_light) v = indptr[L.light0[g] + j] - indptr[L.light0[g]];
    else if (j <= n_light + n_heavy) v = light_nz + indptr[L.heavy0[g] + (j - n_light)] - indptr[L.heavy0[g]];
    else v = light_nz + indptr[L.heavy1[g]] - indptr[L.heavy0[g]];
    out[j] = v;
}

// idx[i] <- position of column idx[i] in the gathered operand; a column outside [0, n) raises the flag
__global__ void __launch_bounds__(256)
dist_relabel_kernel(int *__restrict__ idx, int64_t count, int n, const DistLayout L, int *__restrict__ err_flag)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const int c = idx[i];
        int id = (c >= 0 && c < n) ? dist_new_id(L, c) : -1;
        if (id < 0) { atomicOr(err_flag, 1); id = 0; }
        idx[i] = id;
    }
}

// rows[j] = row of the degree-ordered matrix held at local row j of rank g, or -1 for padding
__global__ void __launch_bounds__(256)
dist_block_rows_kernel(const DistLayout L, int g, int *__restrict__ rows)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= L.per) return;
    const int n_light = L.light1[g] - L.light0[g], n_heavy = L.heavy1[g] - L.heavy0[g];
    rows[j] = j < n_light ? L.light0[g] + j : j < n_light + n_heavy ? L.heavy0[g] + (j - n_light) : -1;
}

}  // namespace agcn
