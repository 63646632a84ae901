// Declarations shared between the translation units of the library (not part of the C ABI).
#pragma once
#include "host_common.h"

struct agcn_spmm_plan {
    const int4 *block4 = nullptr;     // borrowed
    int64_t n_blocks = 0, n_units = 0, n_rows = 0, n_cols = 0, nnz = 0;
    int2 *unit_carry = nullptr;       // [n_units]
    int *carry_row = nullptr;         // [n_carry]
    float *carry = nullptr;           // [n_carry][SPMM_PANEL]
    int *zero_rows = nullptr;         // [n_zero]
    int64_t n_carry = 0, n_zero = 0;
    int launches_last_run = 0;
    int l2_bytes = 0, sm_count = 0;   // of the device the plan was created on
    int panel_override = 0;           // AGCN_SPMM_PANEL at creation (0 = choose automatically)
    bool never_split = false;         // set for the ranges of a column-tiled product
    int batch_override = 0;           // AGCN_SPMM_BATCH at creation: 8 or 16 gathers in flight per lane (experiments)
    int pad_unaligned = 1;            // AGCN_SPMM_PAD at creation: copy unaligned X into 16-byte-aligned rows
    float *x_pad = nullptr;           // [n_cols][dim rounded up to 4], grown on demand
    size_t x_pad_bytes = 0;
};

namespace agcn {

int env_int(const char *name, int dflt);

// partition.cu
int partition_device(const int *d_indptr, int64_t n_rows, int *d_block4, int64_t cap_blocks, int64_t *n_blocks, cudaStream_t s);

// spmm.cu
int spmm_create(agcn_spmm_plan **out, const int *d_block4, int64_t n_blocks, const int *d_indices,
                int64_t n_rows, int64_t n_cols, int64_t nnz, cudaStream_t s);
int spmm_run(agcn_spmm_plan *p, const int *d_indices, const float *d_vals, const float *d_x, int64_t ldx,
             float *d_y, int64_t ldy, int dim, cudaStream_t s, int activation = 0, int accumulate = 0);
int spmm_check_run_args(const agcn_spmm_plan *p, const int *d_indices, const float *d_vals, const float *d_x, int64_t ldx,
                        const float *d_y, int64_t ldy, int dim, int activation);
int spmm_prepare_x(agcn_spmm_plan *p, const float *d_x, int64_t ldx, int dim, cudaStream_t s,
                   const float **x_use, int64_t *ldx_use, bool *x_vec);
// Which part of a product one call of spmm_run_prepared launches.  A product may be issued as
// several unit ranges (a unit = 8 consecutive tuples = one thread block): the zero-fill of
// uncovered rows goes with one of them and the carry kernel, which finishes the heavy rows that
// cross unit boundaries, after the last.
struct SpmmLaunchPart {
    int64_t unit0 = 0, unit1 = -1;      // units [unit0, unit1); -1 = to the end
    bool zero_fill = true, carry = true;
    int64_t carry_s0 = 0, carry_s1 = -1; // carry slots the carry kernel covers (-1 = to the last); row-aligned
    const int *abort_flag = nullptr;    // optional device word: nonzero makes the kernels return at once
    float *carry_buf = nullptr;         // optional carry scratch [n_carry][128] to use instead of the plan's (products in flight together)
};
int spmm_run_prepared(agcn_spmm_plan *p, const int *d_indices, const float *d_vals, const float *x_use, int64_t ldx_use,
                      bool x_vec, float *d_y, int64_t ldy, int dim, cudaStream_t s, int activation, int accumulate,
                      const SpmmLaunchPart &part);
int spmm_check_cols(const int *d_idx, int64_t count, int64_t n_cols, int *d_flag, cudaStream_t s);
void plan_free(agcn_spmm_plan *p);


// gemm.cu: Z = H * W (128 x 128, TF32) enqueued on `s`; nothing allocated, nothing synchronised
int gemm_tf32_async(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz, int64_t m_rows,
                    int *d_status, cudaStream_t s);
// Z2[r] = relu(A[r, :] * Z1) * W for the first m_rows rows of a CSR block, all of at most
// fused_layer_max_degree() nonzeros (gemm.cu)
int fused_layer_async(const int *d_indptr, const int *d_indices, const float *d_vals, const float *d_z_in, const float *d_w,
                      float *d_z_out, int64_t m_rows, int64_t n_cols, int *d_status, cudaStream_t s);
int fused_layer_max_degree();

// layout.cu
int balanced_blocks(const int *h_indptr, int64_t n_rows, int world, int64_t *h_ranges, int64_t *rows_per_block);

}  // namespace agcn
