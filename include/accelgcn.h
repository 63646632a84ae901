/*
 * accelgcn.h -- C ABI of the B200 (sm_100a) implementation of the Accel-GCN
 * hot path: degree sort, block-level partitioning (.block4 metadata) and the
 * block-level-partitioned CSR SpMM  Y = A * X  in fp32.
 *
 * Conventions
 *  - Plain pointers and sizes only.  "d_" parameters are device pointers (or
 *    CUDA managed memory, which the reference harness uses throughout,
 *    main.cu:62-88); "h_" parameters are host pointers.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the default stream).
 *  - Every function returns AGCN_OK (0) or a negative AGCN_ERR_* code and
 *    never aborts; agcn_last_error() gives the message of the calling
 *    thread's last failure.  The caller owns every buffer it passes in; the
 *    library owns only plan-internal scratch.
 *  - All entry points run on the CUDA device that is current in the calling
 *    thread.  There is no CPU fallback: without a usable device the calls
 *    fail with AGCN_ERR_CUDA.
 *  - Reference citations are file:line in xiexi51/ICCAD-Accel-GCN.
 */
#ifndef ACCELGCN_H
#define ACCELGCN_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AGCN_OK             0
#define AGCN_ERR_INVALID   -1   /* bad argument (null pointer, size, alignment) */
#define AGCN_ERR_CUDA      -2   /* a CUDA runtime call failed */
#define AGCN_ERR_CAPACITY  -3   /* output buffer too small; the needed size is reported */
#define AGCN_ERR_RANGE     -4   /* input data out of range (negative degree, bad tuple, bad column) */

/* .block4 format constants (block_level_partition.py:7-8, spmm_accel.cu:11-12) */
#define AGCN_DEG_BOUND        384
#define AGCN_WARPS_PER_BLOCK   12

/* Message of the last error raised on the calling thread ("" if none). */
const char *agcn_last_error(void);

/* Library version: major * 10000 + minor * 100 + patch. */
int agcn_version(void);

/* ------------------------------------------------------------------------
 * Block-level partitioner.
 * Replaces the per-graph body of block_level_partition.py:38-106: row
 * pointers of the (degree-ordered) CSR in, flat int32 4-tuples
 * {block_degree, block_row_begin, block_loc_begin, block_info} out -- the
 * exact contents of block_level_meta/<graph>.block4, bit for bit, for any
 * degree sequence (sorted or not).
 *
 * d_block4 == NULL (or cap_blocks == 0) only counts.  If cap_blocks is too
 * small the call returns AGCN_ERR_CAPACITY with *n_blocks set.  An upper
 * bound that always suffices is  n_rows + nnz / 384.  d_block4 must be
 * 16-byte aligned.  n_rows <= 0 is AGCN_ERR_INVALID (the script raises
 * IndexError on an empty graph, :49); a negative degree is AGCN_ERR_RANGE
 * (the script prints "cur_degree number is wrong" and stops, :98-100).
 * The call returns after the work on `stream` has completed.
 * ---------------------------------------------------------------------- */
int agcn_partition_device(const int32_t *d_indptr, int64_t n_rows,
                          int32_t *d_block4, int64_t cap_blocks, int64_t *n_blocks,
                          void *stream);

/* Same, host buffers in and out (what a ctypes replacement of the script
 * calls after np.fromfile, block_level_partition.py:31-34 / :105-106). */
int agcn_partition_host(const int32_t *h_indptr, int64_t n_rows,
                        int32_t *h_block4, int64_t cap_blocks, int64_t *n_blocks);

/* Partitioner that allocates nothing.  It has no counterpart in the
 * reference; it exists for hosts that cannot let a library call cudaMalloc --
 * processes whose own allocator already owns all device memory, loops that
 * cannot take the device-wide synchronisation an allocation or free implies,
 * plug-in hosts that forbid allocation after start-up.  Same arguments, same
 * results and same error codes as agcn_partition_device, but the tile scratch
 * is a fixed array inside the library's device image (about 96 KB, resident on
 * every GPU that loads the library until the process exits) and the call makes
 * no cudaMalloc / cudaFree or other allocating call.
 *  - n_rows above AGCN_PARTITION_NOALLOC_MAX_ROWS is AGCN_ERR_INVALID.
 *  - The first call on each device looks up the array's device address and, if
 *    it is the library's first launch there, makes the CUDA runtime load the
 *    kernels -- which may itself take device memory.  Make that first call at
 *    start-up, before the host's allocator claims the GPU and before any stream
 *    capture begins; calls after it leave the free-memory figure unchanged.
 *  - All calls on a GPU share the array: calls that overlap on the same GPU
 *    (other streams or threads) race and must be serialised by the caller. */
#define AGCN_PARTITION_NOALLOC_MAX_ROWS 16777216   /* 2^24 */
int agcn_partition_device_noalloc(const int32_t *d_indptr, int64_t n_rows,
                                  int32_t *d_block4, int64_t cap_blocks, int64_t *n_blocks,
                                  void *stream);

/* ------------------------------------------------------------------------
 * Degree sort.
 * Produces the degree-ordered CSR the reference only assumes -- its inputs
 * are pre-sorted <graph>.new_indptr / .new_indices files (main.cu:62-63,
 * block_level_partition.py:31-32, README.md:44-53).  Rows are ordered by
 * ascending degree, ties by ascending original row id (stable).
 *   d_perm[new_row]   = original row            (required, n_rows ints)
 *   d_new_indptr      = row pointers, n_rows+1  (optional)
 *   d_new_indices/d_new_vals = permuted nonzeros (optional; vals only if d_vals)
 * relabel_cols != 0 also renames column ids by the same permutation (new id
 * of original row r = its position in the order), which keeps a square A
 * consistent for multi-layer use; requires every column id < n_rows.
 * Within a row the nonzeros keep their original order.
 * ---------------------------------------------------------------------- */
int agcn_degree_sort_device(const int32_t *d_indptr, const int32_t *d_indices, const float *d_vals,
                            int64_t n_rows, int64_t nnz, int relabel_cols,
                            int32_t *d_perm, int32_t *d_new_indptr,
                            int32_t *d_new_indices, float *d_new_vals, void *stream);

int agcn_degree_sort_host(const int32_t *h_indptr, const int32_t *h_indices, const float *h_vals,
                          int64_t n_rows, int64_t nnz, int relabel_cols,
                          int32_t *h_perm, int32_t *h_new_indptr,
                          int32_t *h_new_indices, float *h_new_vals);

/* ------------------------------------------------------------------------
 * SpMM.
 * Replaces SPMM_ACCEL (spmm_accel.h:4-20): agcn_spmm_create is the per-call
 * preparation of SPMM_ACCEL::do_test (spmm_accel.cu:110-132: load the
 * .block4 array, fix the launch shape), agcn_spmm_run is SPMM_ACCEL::run
 * (spmm_accel.cu:104-108: one asynchronous launch sequence on `stream`, no
 * synchronisation), agcn_spmm_destroy is the cudaFree at :137.
 *
 * The plan borrows d_block4 (it must stay valid and unchanged until
 * destroy).  Creation validates every tuple against n_rows / nnz and, when
 * d_indices is not NULL, every column id against n_cols; bad input gives
 * AGCN_ERR_RANGE instead of a device fault.  Tuples must be in ascending
 * row order, as the partitioner emits them.
 *
 * run:  Y[n_rows x dim] = A * X[n_cols x dim], row-major, row strides ldx /
 * ldy floats (the reference uses ldx = ldy = dim, spmm_accel.cu:75,84).
 * Unlike the reference kernel, which accumulates into Y with atomicAdd for
 * rows of degree >= 33 and never writes rows of degree 0 (:82-98), run
 * overwrites all of Y and does not read it; results are bit-identical from
 * run to run.  Any dim >= 1; the fast path needs dim % 4 == 0, ldx % 4 ==
 * ldy % 4 == 0 and 16-byte aligned d_x / d_y.  dim > 64 may run as two
 * 64-column passes when X is larger than L2 (environment variable
 * AGCN_SPMM_PANEL = columns per pass, read at plan creation, overrides that choice).  A plan must not be run
 * concurrently on two streams (the runs share its carry scratch).
 * ---------------------------------------------------------------------- */
typedef struct agcn_spmm_plan agcn_spmm_plan;

int agcn_spmm_create(agcn_spmm_plan **plan, const int32_t *d_block4, int64_t n_blocks,
                     const int32_t *d_indices, int64_t n_rows, int64_t n_cols, int64_t nnz,
                     void *stream);

int agcn_spmm_run(agcn_spmm_plan *plan, const int32_t *d_indices, const float *d_vals,
                  const float *d_x, int64_t ldx, float *d_y, int64_t ldy, int dim, void *stream);

/* agcn_spmm_run with a fused element-wise activation on Y (the aggregation step of a GCN layer,
 * relu(A * Z)).  The reference kernel has no epilogue; AGCN_ACT_NONE is agcn_spmm_run. */
#define AGCN_ACT_NONE 0
#define AGCN_ACT_RELU 1
int agcn_spmm_run_act(agcn_spmm_plan *plan, const int32_t *d_indices, const float *d_vals,
                      const float *d_x, int64_t ldx, float *d_y, int64_t ldy, int dim, int activation,
                      void *stream);

int agcn_spmm_destroy(agcn_spmm_plan *plan);

/* Number of kernel launches the last agcn_spmm_run on this plan issued, and
 * the sizes of its internal scratch (for reporting). */
int agcn_spmm_plan_info(const agcn_spmm_plan *plan, int64_t *n_units, int64_t *n_carry,
                        int64_t *n_zero_rows, int *launches_last_run);

/* ------------------------------------------------------------------------
 * Dense feature transform of a GCN layer:  Z[m_rows x n_dim] = H[m_rows x k_dim] * W[k_dim x n_dim],
 * row-major fp32 operands, TF32 multiply with fp32 accumulation on the tensor cores (tcgen05).
 * The reference benchmarks the SpMM alone and has no dense transform; this is the X*W step that
 * surrounds it in a GCN layer.  Only k_dim = n_dim = 128 is built (other sizes: AGCN_ERR_INVALID).
 * ldh / ldz are row strides in floats (>= 128, multiples of 4); W is contiguous.  H and Z must be
 * 16-byte aligned and must not overlap.  The call returns after the product has completed.
 * ---------------------------------------------------------------------- */
int agcn_gemm_tf32(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz,
                   int64_t m_rows, int k_dim, int n_dim, void *stream);

/* ------------------------------------------------------------------------
 * Host-buffer SpMM: the plug-in used by a harness that keeps its arrays in
 * host memory.  The split follows SPMM_BASE: agcn_host_set_graph is the
 * constructor's part (spmm_base.h:9-20 takes ptr/idx/val once) plus the
 * .block4 load of do_test (spmm_accel.cu:122) -- it uploads .block4, column
 * ids and values and builds the plan; agcn_host_spmm is one run(dim)
 * (spmm_accel.cu:104-108) on host operands -- it uploads X [n_cols x dim],
 * runs, downloads Y [n_rows x dim] and returns when Y is complete.
 * agcn_spmm_host does both in one call.  The context owns one stream and
 * keeps its device buffers between calls (they only grow).  Host pointers may
 * be pageable or pinned; pinned memory gives full PCIe speed.
 * ---------------------------------------------------------------------- */
typedef struct agcn_host_ctx agcn_host_ctx;

int agcn_host_ctx_create(agcn_host_ctx **ctx);
int agcn_host_ctx_destroy(agcn_host_ctx *ctx);

int agcn_host_set_graph(agcn_host_ctx *ctx, const int32_t *h_block4, int64_t n_blocks,
                        const int32_t *h_indices, const float *h_vals,
                        int64_t n_rows, int64_t n_cols, int64_t nnz);

int agcn_host_spmm(agcn_host_ctx *ctx, const float *h_x, float *h_y, int dim);

int agcn_spmm_host(agcn_host_ctx *ctx, const int32_t *h_block4, int64_t n_blocks,
                   const int32_t *h_indices, const float *h_vals,
                   const float *h_x, float *h_y,
                   int64_t n_rows, int64_t n_cols, int64_t nnz, int dim);

#ifdef __cplusplus
}
#endif
#endif /* ACCELGCN_H */
