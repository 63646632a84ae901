// C-ABI entry points of the column-tiled SpMM (agcn_spmm_tiled_*): A regrouped by column range so
// that every launch gathers from one L2-resident slab of X, each range with its own `.block4`
// metadata from the ordinary partitioner.  The reference gathers un-tiled (spmm_accel.cu:55-78);
// this has no counterpart there.
#include "host_common.h"
#include "internal.h"
#include "kernels/tile_kernels.cuh"

#include <new>
#include <vector>

struct agcn_spmm_tiled {
    int n_ranges = 0;
    int64_t n_rows = 0, n_cols = 0, nnz = 0;
    int *idx = nullptr;                    // [nnz] range-major
    float *val = nullptr;                  // [nnz] range-major
    std::vector<int64_t> first;            // [n_ranges + 1] first nonzero of every range
    std::vector<int *> block4;             // per range, owned
    std::vector<int64_t> n_blocks;
    std::vector<agcn_spmm_plan *> plan;    // per range
    int launches_last_run = 0;
};

namespace agcn {

static void tiled_free(agcn_spmm_tiled *t)
{
    if (t == nullptr) return;
    for (agcn_spmm_plan *p : t->plan) plan_free(p);
    for (int *b : t->block4) cudaFree(b);
    cudaFree(t->idx);
    cudaFree(t->val);
    delete t;
}

static int tiled_create(agcn_spmm_tiled **out, const int *d_indptr, const int *d_indices, const float *d_vals,
                        int64_t n_rows, int64_t n_cols, int64_t nnz, const int *h_bounds, int n_ranges, cudaStream_t s)
{
    AGCN_REQUIRE(out != nullptr, "agcn_spmm_tiled_create: null plan pointer");
    *out = nullptr;
    AGCN_REQUIRE(d_indptr != nullptr && h_bounds != nullptr, "agcn_spmm_tiled_create: null indptr or bounds");
    AGCN_REQUIRE(nnz >= 0 && nnz <= (int64_t)INT32_MAX && (nnz == 0 || (d_indices != nullptr && d_vals != nullptr)),
                 "agcn_spmm_tiled_create: bad nnz, or null indices / values");
    AGCN_REQUIRE(n_rows > 0 && n_rows < (int64_t)INT32_MAX && n_cols > 0 && n_cols < (int64_t)INT32_MAX,
                 "agcn_spmm_tiled_create: n_rows / n_cols out of range");
    AGCN_REQUIRE(n_ranges >= 1 && n_ranges <= TILE_MAX_RANGES, "agcn_spmm_tiled_create: 1..%d column ranges", TILE_MAX_RANGES);
    TileBounds tb;
    tb.n_ranges = n_ranges;
    for (int k = 0; k <= n_ranges; k++) {
        tb.bound[k] = h_bounds[k];
        AGCN_REQUIRE(k == 0 || h_bounds[k] >= h_bounds[k - 1], "agcn_spmm_tiled_create: bounds must not decrease");
    }
    AGCN_REQUIRE(h_bounds[0] == 0 && h_bounds[n_ranges] == n_cols, "agcn_spmm_tiled_create: bounds must run from 0 to n_cols");

    // the caller's nnz sizes the regrouped arrays: it must be the matrix's own count
    int ends[2] = {0, 0};
    AGCN_CUDA(cudaMemcpyAsync(&ends[0], d_indptr, sizeof(int), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaMemcpyAsync(&ends[1], d_indptr + n_rows, sizeof(int), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaStreamSynchronize(s));
    AGCN_REQUIRE(ends[0] == 0 && (int64_t)ends[1] == nnz, "agcn_spmm_tiled_create: indptr must run from 0 to nnz (got %d .. %d, nnz %lld)",
                 ends[0], ends[1], (long long)nnz);

    const int64_t per = n_rows + 1, cells = per * n_ranges;
    DeviceScratch scratch;
    AGCN_ALLOC(count, scratch, int, cells);
    AGCN_ALLOC(position, scratch, int64_t, cells);
    AGCN_ALLOC(tile_sums, scratch, int64_t, scan_tiles(cells));
    AGCN_ALLOC(indptr_t, scratch, int, cells);

    agcn_spmm_tiled *t = new (std::nothrow) agcn_spmm_tiled;
    AGCN_REQUIRE(t != nullptr, "agcn_spmm_tiled_create: out of host memory");
    struct Guard {            // frees the half-built plan on every early return
        agcn_spmm_tiled *t;
        ~Guard() { tiled_free(t); }
    } guard{t};
    t->n_ranges = n_ranges; t->n_rows = n_rows; t->n_cols = n_cols; t->nnz = nnz;
    t->first.assign(n_ranges + 1, 0);
    t->block4.assign(n_ranges, nullptr);
    t->n_blocks.assign(n_ranges, 0);
    t->plan.assign(n_ranges, nullptr);

    if (nnz > 0) {
        AGCN_CUDA(cudaMalloc(&t->idx, (size_t)nnz * sizeof(int)));
        AGCN_CUDA(cudaMalloc(&t->val, (size_t)nnz * sizeof(float)));
    }
    const unsigned row_grid = (unsigned)ceil_div(per, TILE_WARPS);
    AGCN_KERNEL(tile_count_kernel, row_grid, TILE_WARPS * 32, s, d_indptr, d_indices, n_rows, tb, count);
    AGCN_LAUNCH_CHECK("tile_count_kernel");
    int rc = exclusive_scan_i32_i64(count, position, cells, tile_sums, nullptr, s);
    if (rc != AGCN_OK) return rc;
    if (nnz > 0) {
        AGCN_KERNEL(tile_place_kernel, row_grid, TILE_WARPS * 32, s, d_indptr, d_indices, d_vals, n_rows, tb,
                    (const int64_t *)position, t->idx, t->val);
        AGCN_LAUNCH_CHECK("tile_place_kernel");
    }
    AGCN_KERNEL(tile_indptr_kernel, (unsigned)ceil_div(cells, 256), 256, s, (const int64_t *)position, n_rows, n_ranges, indptr_t);
    AGCN_LAUNCH_CHECK("tile_indptr_kernel");
    // first nonzero of every range: position of (range k, row 0)
    for (int k = 0; k < n_ranges; k++)
        AGCN_CUDA(cudaMemcpyAsync(&t->first[k], position + (int64_t)k * per, sizeof(int64_t), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaStreamSynchronize(s));
    t->first[n_ranges] = nnz;

    // every range is an ordinary CSR matrix over all rows: ordinary partitioner, ordinary plan
    for (int k = 0; k < n_ranges; k++) {
        const int *ip_k = indptr_t + (int64_t)k * per;
        const int64_t nnz_k = t->first[k + 1] - t->first[k];
        int64_t nb = 0;
        rc = partition_device(ip_k, n_rows, nullptr, 0, &nb, s);
        if (rc != AGCN_OK) return rc;
        if (nb > 0) {
            AGCN_CUDA(cudaMalloc(&t->block4[k], (size_t)nb * 16));
            rc = partition_device(ip_k, n_rows, t->block4[k], nb, &nb, s);
            if (rc != AGCN_OK) return rc;
        }
        t->n_blocks[k] = nb;
        rc = spmm_create(&t->plan[k], t->block4[k], nb, nnz_k > 0 ? t->idx + t->first[k] : nullptr, n_rows, n_cols, nnz_k, s);
        if (rc != AGCN_OK) return rc;
        t->plan[k]->never_split = true;      // a range's slab stays in L2 by construction: no column passes
    }
    guard.t = nullptr;
    *out = t;
    return AGCN_OK;
}

static int tiled_run(agcn_spmm_tiled *t, int k0, int k1, const float *d_x, int64_t ldx, float *d_y, int64_t ldy, int dim,
                     int activation, cudaStream_t s)
{
    AGCN_REQUIRE(t != nullptr, "agcn_spmm_tiled_run: null plan");
    AGCN_REQUIRE(k0 >= 0 && k0 < k1 && k1 <= t->n_ranges, "agcn_spmm_tiled_run: range %d..%d outside 0..%d", k0, k1, t->n_ranges);
    agcn_spmm_plan *p0 = t->plan[k0];
    int rc = spmm_check_run_args(p0, t->idx, t->val, d_x, ldx, d_y, ldy, dim, activation);
    if (rc != AGCN_OK) return rc;
    if (k0 == 0) t->launches_last_run = 0;
    // an unaligned X is copied to aligned rows once, by the first range's plan, for all ranges of the call
    const float *x_use = nullptr;
    int64_t ldx_use = 0;
    bool x_vec = false;
    p0->launches_last_run = 0;
    rc = spmm_prepare_x(p0, d_x, ldx, dim, s, &x_use, &ldx_use, &x_vec);
    if (rc != AGCN_OK) return rc;
    t->launches_last_run += p0->launches_last_run;
    for (int k = k0; k < k1; k++) {
        agcn_spmm_plan *p = t->plan[k];
        p->launches_last_run = 0;
        const int64_t off = t->first[k];
        // the first range stores Y (and zero-fills rows it does not cover), later ranges add to it in
        // range order; the activation is applied by the last range, to every row
        rc = spmm_run_prepared(p, t->idx + off, t->val + off, x_use, ldx_use, x_vec, d_y, ldy, dim, s,
                               k == t->n_ranges - 1 ? activation : 0, k > 0 ? 1 : 0, SpmmLaunchPart());
        if (rc != AGCN_OK) return rc;
        t->launches_last_run += p->launches_last_run;
    }
    return AGCN_OK;
}

}  // namespace agcn

extern "C" int agcn_spmm_tiled_create(agcn_spmm_tiled **plan, const int32_t *d_indptr, const int32_t *d_indices,
                                      const float *d_vals, int64_t n_rows, int64_t n_cols, int64_t nnz,
                                      const int32_t *h_bounds, int n_ranges, void *stream)
{
    agcn::clear_error();
    return agcn::tiled_create(plan, d_indptr, d_indices, d_vals, n_rows, n_cols, nnz, h_bounds, n_ranges,
                              static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_spmm_tiled_run(agcn_spmm_tiled *plan, const float *d_x, int64_t ldx, float *d_y, int64_t ldy, int dim,
                                   int activation, void *stream)
{
    agcn::clear_error();
    AGCN_REQUIRE(plan != nullptr, "agcn_spmm_tiled_run: null plan");
    return agcn::tiled_run(plan, 0, plan->n_ranges, d_x, ldx, d_y, ldy, dim, activation, static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_spmm_tiled_run_range(agcn_spmm_tiled *plan, int range, const float *d_x, int64_t ldx, float *d_y,
                                         int64_t ldy, int dim, int activation, void *stream)
{
    agcn::clear_error();
    return agcn::tiled_run(plan, range, range + 1, d_x, ldx, d_y, ldy, dim, activation, static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_spmm_tiled_destroy(agcn_spmm_tiled *plan)
{
    agcn::clear_error();
    agcn::tiled_free(plan);
    return AGCN_OK;
}

extern "C" int agcn_spmm_tiled_info(const agcn_spmm_tiled *plan, int *n_ranges, int64_t *n_blocks_total, int64_t *range_nnz,
                                    int *launches_last_run)
{
    agcn::clear_error();
    AGCN_REQUIRE(plan != nullptr, "agcn_spmm_tiled_info: null plan");
    if (n_ranges) *n_ranges = plan->n_ranges;
    if (n_blocks_total) {
        *n_blocks_total = 0;
        for (int64_t nb : plan->n_blocks) *n_blocks_total += nb;
    }
    if (range_nnz)
        for (int k = 0; k < plan->n_ranges; k++) range_nnz[k] = plan->first[k + 1] - plan->first[k];
    if (launches_last_run) *launches_last_run = plan->launches_last_run;
    return AGCN_OK;
}

// How many column ranges a product of this shape should be cut into (1 = do not tile).
// A slab of X (range columns x dim x 4 bytes) should stay in L2 next to the streams of A and Y
// passing through: about a third of L2 per slab.  Tiling pays only while every row keeps enough
// nonzeros per range to amortise the extra pass over Y (read + write per range after the first):
// a mean of 48 per row and range.
extern "C" int agcn_spmm_tiled_suggest(int64_t n_rows, int64_t n_cols, int64_t nnz, int dim)
{
    int dev = 0, l2 = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev) != cudaSuccess || l2 <= 0)
        return 1;
    if (n_rows <= 0 || n_cols <= 0 || dim <= 0) return 1;
    const double x_bytes = (double)n_cols * dim * 4.0;
    if (x_bytes <= 0.6 * l2) return 1;
    int k = (int)((x_bytes + 0.35 * l2 - 1.0) / (0.35 * l2));
    if (k > agcn::TILE_MAX_RANGES) k = agcn::TILE_MAX_RANGES;
    while (k > 1 && (double)nnz / (double)n_rows / k < 48.0) k--;
    return k;
}
