// C-ABI entry points of the degree sort (the ordering the reference assumes
// of its <graph>.new_indptr / .new_indices inputs, main.cu:62-63).
#include "host_common.h"
#include "kernels/degree_sort_kernels.cuh"

#include <utility>

namespace agcn {

static int degree_sort_device(const int *d_indptr, const int *d_indices, const float *d_vals,
                              int64_t n_rows, int64_t nnz, int relabel_cols,
                              int *d_perm, int *d_new_indptr, int *d_new_indices, float *d_new_vals,
                              cudaStream_t s)
{
    AGCN_REQUIRE(d_indptr != nullptr && d_perm != nullptr, "agcn_degree_sort: null indptr or perm");
    AGCN_REQUIRE(n_rows > 0 && n_rows < (int64_t)INT32_MAX, "agcn_degree_sort: n_rows = %lld out of range", (long long)n_rows);
    AGCN_REQUIRE(nnz >= 0 && nnz <= (int64_t)INT32_MAX, "agcn_degree_sort: nnz = %lld out of range", (long long)nnz);
    AGCN_REQUIRE(d_new_indices == nullptr || d_indices != nullptr, "agcn_degree_sort: new_indices wanted but indices is null");
    AGCN_REQUIRE(d_new_vals == nullptr || (d_vals != nullptr && d_new_indices != nullptr),
                 "agcn_degree_sort: new_vals needs vals and new_indices");
    AGCN_REQUIRE(d_new_indices == nullptr || d_new_indptr != nullptr, "agcn_degree_sort: new_indices needs new_indptr");

    const int64_t tiles = ceil_div(n_rows, SORT_TILE);
    const int64_t hist_len = tiles * RADIX_BINS;
    DeviceScratch scratch;
    AGCN_ALLOC(keys_a, scratch, unsigned, n_rows + 1);
    AGCN_ALLOC(keys_b, scratch, unsigned, n_rows + 1);
    AGCN_ALLOC(rows_a, scratch, int, n_rows);
    AGCN_ALLOC(rows_b, scratch, int, n_rows);
    AGCN_ALLOC(hist, scratch, unsigned, hist_len);
    AGCN_ALLOC(hist_scanned, scratch, unsigned, hist_len);
    AGCN_ALLOC(scan_sums, scratch, unsigned, scan_tiles(hist_len > n_rows + 1 ? hist_len : n_rows + 1));
    AGCN_ALLOC(d_flags, scratch, int, 2);   // [0] max degree, [1] error flag
    AGCN_CUDA(cudaMemsetAsync(d_flags, 0, 2 * sizeof(int), s));

    AGCN_KERNEL(degree_keys_kernel, (unsigned)ceil_div(n_rows, 256 * KEYS_ITEMS), 256, s, d_indptr, n_rows, keys_a, rows_a, d_flags, d_flags + 1);
    AGCN_LAUNCH_CHECK("degree_keys_kernel");
    int flags[2] = {0, 0}, ends[2] = {0, 0};
    AGCN_CUDA(cudaMemcpyAsync(flags, d_flags, sizeof(flags), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaMemcpyAsync(&ends[0], d_indptr, sizeof(int), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaMemcpyAsync(&ends[1], d_indptr + n_rows, sizeof(int), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaStreamSynchronize(s));
    if (flags[1] != 0) {
        set_error("agcn_degree_sort: indptr decreases somewhere (negative degree)");
        return AGCN_ERR_RANGE;
    }
    // the caller's nnz sizes the grid of the CSR permute: it must be the matrix's own count
    if (d_new_indices != nullptr && (int64_t)ends[1] - (int64_t)ends[0] != nnz) {
        set_error("agcn_degree_sort: nnz = %lld but indptr[n_rows] - indptr[0] = %lld", (long long)nnz,
                  (long long)ends[1] - (long long)ends[0]);
        return AGCN_ERR_INVALID;
    }
    int bits = 0;
    while (bits < 32 && (flags[0] >> bits) != 0) bits++;

    unsigned *keys_in = keys_a, *keys_out = keys_b;
    int *rows_in = rows_a, *rows_out = rows_b;
    for (int shift = 0; shift < bits; shift += RADIX_BITS) {
        AGCN_KERNEL(radix_histogram_kernel, (unsigned)tiles, SORT_BLOCK, s, (const unsigned *)keys_in, n_rows, shift, tiles, hist);
        AGCN_LAUNCH_CHECK("radix_histogram_kernel");
        int rc = exclusive_scan_u32_u32(hist, hist_scanned, hist_len, scan_sums, s);
        if (rc != AGCN_OK) return rc;
        AGCN_KERNEL(radix_scatter_kernel, (unsigned)tiles, SORT_BLOCK, s, (const unsigned *)keys_in, (const int *)rows_in,
                    n_rows, shift, tiles, (const unsigned *)hist_scanned, keys_out, rows_out);
        AGCN_LAUNCH_CHECK("radix_scatter_kernel");
        std::swap(keys_in, keys_out);
        std::swap(rows_in, rows_out);
    }
    // keys_in = ascending degrees, rows_in = perm
    AGCN_CUDA(cudaMemcpyAsync(d_perm, rows_in, (size_t)n_rows * sizeof(int), cudaMemcpyDeviceToDevice, s));
    if (d_new_indptr != nullptr) {
        AGCN_CUDA(cudaMemsetAsync(keys_in + n_rows, 0, sizeof(unsigned), s));
        int rc = exclusive_scan_u32_i32(keys_in, d_new_indptr, n_rows + 1, reinterpret_cast<int *>(scan_sums), s);
        if (rc != AGCN_OK) return rc;
    }
    if (d_new_indices != nullptr && nnz > 0) {
        int *new_id = nullptr;
        if (relabel_cols) {
            new_id = rows_out;   // free after the last pass
            AGCN_KERNEL(invert_perm_kernel, (unsigned)ceil_div(n_rows, 256), 256, s, (const int *)rows_in, n_rows, new_id);
            AGCN_LAUNCH_CHECK("invert_perm_kernel");
        }
        AGCN_KERNEL(csr_permute_kernel, (unsigned)ceil_div(nnz, PERMUTE_TILE), PERMUTE_BLOCK, s,
                    d_indptr, d_indices, d_new_vals != nullptr ? d_vals : (const float *)nullptr, (const int *)rows_in, (const int *)d_new_indptr, (const int *)new_id,
                    n_rows, nnz, d_new_indices, d_new_vals, d_flags + 1);
        AGCN_LAUNCH_CHECK("csr_permute_kernel");
        AGCN_CUDA(cudaMemcpyAsync(flags, d_flags, sizeof(flags), cudaMemcpyDeviceToHost, s));
    }
    AGCN_CUDA(cudaStreamSynchronize(s));
    if (flags[1] != 0) {
        set_error("agcn_degree_sort: a column id lies outside [0, n_rows) and cannot be relabelled");
        return AGCN_ERR_RANGE;
    }
    return AGCN_OK;
}

}  // namespace agcn

extern "C" int agcn_degree_sort_device(const int32_t *d_indptr, const int32_t *d_indices, const float *d_vals,
                                       int64_t n_rows, int64_t nnz, int relabel_cols,
                                       int32_t *d_perm, int32_t *d_new_indptr,
                                       int32_t *d_new_indices, float *d_new_vals, void *stream)
{
    agcn::clear_error();
    return agcn::degree_sort_device(d_indptr, d_indices, d_vals, n_rows, nnz, relabel_cols, d_perm, d_new_indptr,
                                    d_new_indices, d_new_vals, static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_degree_sort_host(const int32_t *h_indptr, const int32_t *h_indices, const float *h_vals,
                                     int64_t n_rows, int64_t nnz, int relabel_cols,
                                     int32_t *h_perm, int32_t *h_new_indptr,
                                     int32_t *h_new_indices, float *h_new_vals)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(h_indptr != nullptr && h_perm != nullptr, "agcn_degree_sort_host: null indptr or perm");
    AGCN_REQUIRE(n_rows > 0 && nnz >= 0, "agcn_degree_sort_host: bad sizes");
    const bool want_idx = h_new_indices != nullptr, want_val = h_new_vals != nullptr;
    AGCN_REQUIRE(!want_idx || (h_indices != nullptr && h_new_indptr != nullptr), "agcn_degree_sort_host: new_indices needs indices and new_indptr");
    AGCN_REQUIRE(!want_val || (h_vals != nullptr && want_idx), "agcn_degree_sort_host: new_vals needs vals and new_indices");
    DeviceScratch scratch;
    AGCN_ALLOC(d_indptr, scratch, int, n_rows + 1);
    AGCN_ALLOC(d_perm, scratch, int, n_rows);
    AGCN_ALLOC(d_new_indptr, scratch, int, n_rows + 1);
    int *d_indices = nullptr, *d_new_indices = nullptr;
    float *d_vals = nullptr, *d_new_vals = nullptr;
    AGCN_CUDA(cudaMemcpy(d_indptr, h_indptr, (size_t)(n_rows + 1) * sizeof(int), cudaMemcpyHostToDevice));
    if (want_idx) {
        d_indices = scratch.alloc<int>(nnz);
        d_new_indices = scratch.alloc<int>(nnz);
        if (d_indices == nullptr || d_new_indices == nullptr) return AGCN_ERR_CUDA;
        AGCN_CUDA(cudaMemcpy(d_indices, h_indices, (size_t)nnz * sizeof(int), cudaMemcpyHostToDevice));
    }
    if (want_val) {
        d_vals = scratch.alloc<float>(nnz);
        d_new_vals = scratch.alloc<float>(nnz);
        if (d_vals == nullptr || d_new_vals == nullptr) return AGCN_ERR_CUDA;
        AGCN_CUDA(cudaMemcpy(d_vals, h_vals, (size_t)nnz * sizeof(float), cudaMemcpyHostToDevice));
    }
    int rc = degree_sort_device(d_indptr, d_indices, d_vals, n_rows, nnz, relabel_cols, d_perm, d_new_indptr,
                                d_new_indices, d_new_vals, nullptr);
    if (rc != AGCN_OK) return rc;
    AGCN_CUDA(cudaMemcpy(h_perm, d_perm, (size_t)n_rows * sizeof(int), cudaMemcpyDeviceToHost));
    if (h_new_indptr != nullptr)
        AGCN_CUDA(cudaMemcpy(h_new_indptr, d_new_indptr, (size_t)(n_rows + 1) * sizeof(int), cudaMemcpyDeviceToHost));
    if (want_idx && nnz > 0)
        AGCN_CUDA(cudaMemcpy(h_new_indices, d_new_indices, (size_t)nnz * sizeof(int), cudaMemcpyDeviceToHost));
    if (want_val && nnz > 0)
        AGCN_CUDA(cudaMemcpy(h_new_vals, d_new_vals, (size_t)nnz * sizeof(float), cudaMemcpyDeviceToHost));
    return AGCN_OK;
}
