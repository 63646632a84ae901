/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement (oracle) of the Accel-GCN SpMM
 * kernel and of the CSR x dense product it is checked against.  Nothing in
 * the product library links, loads or calls this file; only the test-suite,
 * the smoke check and the CPU-baseline leg of the benchmark do.
 *
 * Parity status: the reference ships no golden output vectors for the SpMM
 * (its only check is an in-harness comparison with cuSPARSE, main.cu:141-156).
 * This restatement is therefore pinned two ways: (i) against scipy's
 * CSR @ dense product in float64 on the same inputs, and (ii) on a GPU box,
 * against the reference's own kernel compiled from its sources
 * (oracle/_ref).  Tolerance used everywhere: rel 1e-4 / abs 1e-5 in fp32.
 *
 * Reference followed: spmm_accel.cu
 *   :18-34  block decode           :36-53  combined-warp mapping
 *   :55-78  gather / FMA loop      :82-99  write-back (store vs atomicAdd)
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_DEG_BOUND 384        /* spmm_accel.cu:11 */
#define ORACLE_WARPS_PER_BLOCK 12   /* spmm_accel.cu:12 */

/* One thread-block of the reference kernel per .block4 entry, executed
 * sequentially: entry by entry, virtual warp by virtual warp, lane by lane.
 * Within a virtual warp the <= w_nz products are accumulated in fp32 in index
 * order (spmm_accel.cu:56-78); virtual warps that share a row add their
 * partial to Y (the kernel's atomicAdd, :82-86 and :95-98 -- here in
 * ascending warp order, one of the orders the GPU may take), and rows of
 * degree <= 32 are stored (:89-93).  As in the reference, Y must be zero on
 * entry for rows of degree >= 33 to come out right, and rows of degree 0 are
 * never written.  Offsets are 64-bit here (the reference's are int).
 * Returns 0, or -1 if an index is out of range. */
int agcn_oracle_spmm_block4(const int32_t *block4, int64_t n_blocks,
                            const int32_t *idx, const float *val,
                            const float *x, float *y,
                            int64_t n_rows, int64_t n_cols, int64_t nnz, int dim)
{
    for (int64_t b = 0; b < n_blocks; b++) {
        const int32_t deg = block4[4 * b + 0], row0 = block4[4 * b + 1];
        const int32_t loc0 = block4[4 * b + 2], info = block4[4 * b + 3];
        const int small = deg <= ORACLE_DEG_BOUND;
        const int rows_here = small ? (info & 65535) : 1;                       /* :26 */
        const int w_nz = small ? (info >> 16) : ORACLE_DEG_BOUND / ORACLE_WARPS_PER_BLOCK; /* :27 */
        const int row_nz = small ? deg : info;                                  /* :28 */
        if (w_nz <= 0) return -1;
        const int warps_per_row = (row_nz + w_nz - 1) / w_nz;                   /* :34 */
        for (int wid = 0; wid < ORACLE_WARPS_PER_BLOCK; wid++) {
            const int r = wid / warps_per_row;                                  /* :47 */
            const int c0 = (wid % warps_per_row) * w_nz;                        /* :48 */
            if (r >= rows_here) continue;                                       /* :50-53 */
            if (c0 >= row_nz) continue;    /* out_cache never initialised; nothing accumulated */
            const int64_t out_row = (int64_t)row0 + (warps_per_row > 1 ? r : wid);
            if (out_row < 0 || out_row >= n_rows) return -1;
            for (int lane = 0; lane < dim; lane++) {
                float acc = 0.0f;
                for (int i = 0; i < w_nz && i + c0 < row_nz; i++) {
                    const int64_t p = (int64_t)loc0 + (int64_t)r * row_nz + i + c0;     /* :71 */
                    if (p < 0 || p >= nnz) return -1;
                    const int64_t c = idx[p];
                    if (c < 0 || c >= n_cols) return -1;
                    acc += val[p] * x[c * dim + lane];                                  /* :72-76 */
                }
                float *dst = &y[out_row * dim + lane];
                if (warps_per_row > 1)      *dst += acc;          /* :82-86 */
                else if (small)             *dst = acc;           /* :89-93 */
                else                        *dst += acc;          /* :95-98 */
            }
        }
    }
    return 0;
}

/* Plain CSR x dense, fp64 accumulation, fp32 result: the arithmetic of the
 * check the reference harness makes with cusparseSpMM (spmm_cusparse.cu:6-62,
 * CSR, row-major dense, alpha=1, beta=0), restated on the CPU.  Overwrites
 * all of Y.  Rows are spread over the OpenMP threads available. */
int agcn_oracle_spmm_csr_f64acc(const int32_t *indptr, const int32_t *idx, const float *val,
                                const float *x, float *y,
                                int64_t n_rows, int64_t n_cols, int dim)
{
    int bad = 0;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t r = 0; r < n_rows; r++) {
        double acc[512];
        for (int d0 = 0; d0 < dim; d0 += 512) {
            const int w = dim - d0 < 512 ? dim - d0 : 512;
            for (int k = 0; k < w; k++) acc[k] = 0.0;
            for (int64_t p = indptr[r]; p < indptr[r + 1]; p++) {
                const int64_t c = idx[p];
                if (c < 0 || c >= n_cols) { bad = 1; continue; }
                const double a = val[p];
                const float *xr = x + c * dim + d0;
                for (int k = 0; k < w; k++) acc[k] += a * (double)xr[k];
            }
            for (int k = 0; k < w; k++) y[r * dim + d0 + k] = (float)acc[k];
        }
    }
    return bad ? -1 : 0;
}

/* CSR x dense in fp32 (the precision the reference computes in), rows spread
 * over all OpenMP threads: the CPU baseline that is timed beside the GPU
 * kernel.  Same arithmetic as scipy's csr @ dense for float32 operands. */
int agcn_oracle_spmm_csr_f32(const int32_t *indptr, const int32_t *idx, const float *val,
                             const float *x, float *y,
                             int64_t n_rows, int64_t n_cols, int dim)
{
    (void)n_cols;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t r = 0; r < n_rows; r++) {
        float *yr = y + r * dim;
        for (int k = 0; k < dim; k++) yr[k] = 0.0f;
        for (int64_t p = indptr[r]; p < indptr[r + 1]; p++) {
            const float a = val[p];
            const float *xr = x + (int64_t)idx[p] * dim;
            for (int k = 0; k < dim; k++) yr[k] += a * xr[k];
        }
    }
    return 0;
}

/* Use n OpenMP threads from now on (launchers such as torchrun export OMP_NUM_THREADS=1). */
void agcn_oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int agcn_oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
