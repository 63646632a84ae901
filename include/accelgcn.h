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
 * run to run.  Any dim >= 1 (the reference harness sweeps every dim 16..128,
 * main.cu:12,137).  Rows of X are gathered 16 bytes per lane; when they are not
 * 16-byte aligned (dim % 4 != 0 with ld = dim, an odd stride or base) X is first
 * copied into plan-owned aligned rows (grown on demand: the first such call of
 * a width allocates; AGCN_SPMM_PAD=0 at plan creation selects 4-byte gathers
 * instead) and unaligned rows of Y get element-wise stores.  dim > 64 may run
 * as two 64-column passes when X is larger than L2 (environment variable
 * AGCN_SPMM_PANEL = columns per pass, read at plan creation, overrides that
 * choice).  A plan must not be run concurrently on two streams (the runs share
 * its scratch).
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
 * Column-tiled SpMM.  No counterpart in the reference, whose kernel gathers X
 * un-tiled (spmm_accel.cu:55-78).  The gather runs at L2 speed only while the
 * rows of X it touches stay in L2.  For an X larger than that, A's columns are
 * cut into ranges [h_bounds[k], h_bounds[k+1]) whose slab of X fits, the
 * nonzeros are regrouped range by range (a second copy of A owned by the plan,
 * original order kept inside every row), and each range gets ordinary .block4
 * metadata from the ordinary partitioner (the format is untouched).  A run
 * multiplies range after range: the first stores Y, the later ones add to it in
 * range order, so A is streamed once in total, every launch touches one slab of
 * X, and results are bit-identical from run to run (they differ from the
 * un-tiled product only in the order of the fp32 additions).
 * create: d_indptr / d_indices / d_vals are the CSR arrays (indptr from 0 to
 * nnz); h_bounds is a HOST array of n_ranges + 1 ascending column ids from 0 to
 * n_cols, n_ranges <= 32.  run_range multiplies one range (range 0 stores, any
 * other adds; `activation` is applied only when `range` is the last one), for
 * callers that produce X slab by slab -- ranges must be run in ascending order.
 * agcn_spmm_tiled_suggest returns how many equal ranges a product of that shape
 * should use on the current device (1 = do not tile).
 * ---------------------------------------------------------------------- */
typedef struct agcn_spmm_tiled agcn_spmm_tiled;

int agcn_spmm_tiled_create(agcn_spmm_tiled **plan, const int32_t *d_indptr, const int32_t *d_indices,
                           const float *d_vals, int64_t n_rows, int64_t n_cols, int64_t nnz,
                           const int32_t *h_bounds, int n_ranges, void *stream);
int agcn_spmm_tiled_run(agcn_spmm_tiled *plan, const float *d_x, int64_t ldx, float *d_y, int64_t ldy,
                        int dim, int activation, void *stream);
int agcn_spmm_tiled_run_range(agcn_spmm_tiled *plan, int range, const float *d_x, int64_t ldx,
                              float *d_y, int64_t ldy, int dim, int activation, void *stream);
int agcn_spmm_tiled_destroy(agcn_spmm_tiled *plan);
/* range_nnz, if not NULL, receives n_ranges values */
int agcn_spmm_tiled_info(const agcn_spmm_tiled *plan, int *n_ranges, int64_t *n_blocks_total,
                         int64_t *range_nnz, int *launches_last_run);
int agcn_spmm_tiled_suggest(int64_t n_rows, int64_t n_cols, int64_t nnz, int dim);

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

/* The same product enqueued on `stream` without waiting and without allocating: the form a layer
 * loop uses (the next kernel or collective is enqueued behind it).  d_status is a device int32
 * the caller owns; it is zeroed on the stream before the kernel and holds 0 afterwards unless a
 * bounded pipeline wait inside the kernel ran out (1 = TMA producer, 2 = MMA issuer,
 * 3 = epilogue), in which case Z is incomplete.  Read it at the caller's next synchronisation. */
int agcn_gemm_tf32_async(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz,
                         int64_t m_rows, int k_dim, int n_dim, int32_t *d_status, void *stream);

/* Self-test of the kernel's failure path (no other use): runs the product with a spin limit of
 * well under a millisecond and with the first load of every thread block left out, so that one
 * pipeline wait must run out.  The kernel leaves through its abort path (tensor memory freed,
 * nothing traps or hangs) and the call returns AGCN_ERR_CUDA; AGCN_OK would mean the wait did not
 * run out.  The device stays usable: the next agcn_gemm_tf32 must succeed. */
int agcn_gemm_tf32_selftest_timeout(const float *d_h, int64_t ldh, const float *d_w, float *d_z,
                                    int64_t ldz, int64_t m_rows, void *stream);

/* One GCN layer boundary in one kernel, for rows of at most 32 nonzeros (no counterpart in the
 * reference, which stops at the SpMM, spmm_accel.cu:104-108):
 *     Z2[r, :] = relu(A[r, :] * Z1) * W      for r in [0, m_rows)
 * A is given by its CSR arrays (d_indptr int32[>= m_rows + 1], d_indices / d_vals); EVERY one of these
 * rows must have at most 32 nonzeros -- the leading rows of a degree-ordered matrix -- or the
 * result of a longer row is wrong (the kernel uses its first 32 nonzeros only; it does not fault):
 * callers check the degree of row m_rows - 1.  Z1 is [n_cols x 128] and W [128 x 128], row-major,
 * Z2 [m_rows x 128]; TF32 multiply with fp32 accumulation for the dense part, fp32 for the sparse part.
 * The activations relu(A * Z1) are gathered straight into the shared-memory operand tiles of the
 * tensor-core product and never reach global memory.  Asynchronous; d_status as in agcn_gemm_tf32_async,
 * plus 4 = a column id outside [0, n_cols) was met (that nonzero was read from row 0: no fault). */
int agcn_gcn_fused_layer(const int32_t *d_indptr, const int32_t *d_indices, const float *d_vals,
                         const float *d_z_in, const float *d_w, float *d_z_out, int64_t m_rows,
                         int64_t n_cols, int32_t *d_status, void *stream);

/* ------------------------------------------------------------------------
 * Host-buffer SpMM: the plug-in used by a harness that keeps its arrays in
 * host memory.  The split follows SPMM_BASE: agcn_host_set_graph is the
 * constructor's part (spmm_base.h:9-20 takes ptr/idx/val once) plus the
 * .block4 load of do_test (spmm_accel.cu:122) -- it uploads .block4, column
 * ids and values and builds the plan; agcn_host_spmm is one run(dim)
 * (spmm_accel.cu:104-108) on host operands -- it uploads X [n_cols x dim],
 * runs, downloads Y [n_rows x dim] and returns when Y is complete.
 * agcn_spmm_host does both in one call.  The context owns three streams
 * (upload, kernels, download) and keeps its device buffers between calls (they
 * only grow).  Host pointers may be pageable or pinned; pinned memory gives
 * full PCIe speed and lets the three streams overlap.
 * ---------------------------------------------------------------------- */
typedef struct agcn_host_ctx agcn_host_ctx;

int agcn_host_ctx_create(agcn_host_ctx **ctx);
int agcn_host_ctx_destroy(agcn_host_ctx *ctx);

int agcn_host_set_graph(agcn_host_ctx *ctx, const int32_t *h_block4, int64_t n_blocks,
                        const int32_t *h_indices, const float *h_vals,
                        int64_t n_rows, int64_t n_cols, int64_t nnz);

int agcn_host_spmm(agcn_host_ctx *ctx, const float *h_x, float *h_y, int dim);

/* Several run(dim) calls enqueued together (what one pass of the harness loop over its widths
 * does, main.cu:137-167): product i is Y_i[n_rows x dims[i]] = A * X_i[n_cols x dims[i]].  The
 * upload of X_{i+1}, the kernels of product i and the download of Y_i run concurrently, and a
 * product's rows are downloaded range by range while later ranges are still being computed.
 * Returns when every Y_i is complete.  Results are bit-identical to agcn_host_spmm. */
int agcn_host_spmm_batch(agcn_host_ctx *ctx, int n_products, const float *const *h_x,
                         float *const *h_y, const int *dims);

int agcn_spmm_host(agcn_host_ctx *ctx, const int32_t *h_block4, int64_t n_blocks,
                   const int32_t *h_indices, const float *h_vals,
                   const float *h_x, float *h_y,
                   int64_t n_rows, int64_t n_cols, int64_t nnz, int dim);

/* agcn_host_set_graph + agcn_host_spmm_batch in one call, for a harness that hands over the
 * graph with every step.  Column ids and values go up in ranges of tuples, and every range is
 * multiplied for all products as soon as it has arrived, so kernels and downloads hide under
 * the upload of A (dims that are multiples of 4 up to 128; other widths upload first, then
 * multiply).  A column id outside [0, n_cols) is found by a check that runs ahead of each
 * range's kernels and stops them: the call returns AGCN_ERR_RANGE and the Y_i are undefined. */
int agcn_spmm_host_batch(agcn_host_ctx *ctx, const int32_t *h_block4, int64_t n_blocks,
                         const int32_t *h_indices, const float *h_vals,
                         int64_t n_rows, int64_t n_cols, int64_t nnz,
                         int n_products, const float *const *h_x, float *const *h_y, const int *dims);

/* Where the time of the last agcn_spmm_host_batch call on this context went (the streamed form:
 * every width a multiple of 4 up to 128), in milliseconds from the start of its uploads:
 * ms6[0] last byte of A uploaded, [1] first kernel started, [2] last kernel finished, [3] last
 * byte of Y downloaded; host side: [4] until the plan was built, [5] until all was enqueued. */
int agcn_host_last_timing(agcn_host_ctx *ctx, float *ms6);

/* ------------------------------------------------------------------------
 * Row-sharded multi-GPU SpMM.  The reference is single-GPU (main.cu:53-182);
 * this applies its operator block by block, one caller (process or thread) per
 * GPU, with one exchange per product: the all-gather of the dense operand
 * (NCCL, bound at run time from libnccl.so.2; a single rank never loads it).
 *
 * Layout.  agcn_balanced_blocks (host only: no device is needed) gives every
 * rank TWO ranges of the degree-ordered rows, [light_begin, light_end) from the
 * light end and [heavy_begin, heavy_end) from the heavy end, such that each rank
 * holds rows_per_block = ceil(n_rows / world) rows (the last blocks may be
 * short) and about nnz / world nonzeros: the SpMM, the dense transform and the
 * all-gather are all balanced (cutting contiguous ranges by nonzeros alone
 * leaves one rank with most of the rows and most of the exchange to send).
 * h_ranges receives world x 4 row ids.  Rank g's local row j is row
 * light_begin + j of the matrix for j < light_end - light_begin, then the heavy
 * rows, then empty padding rows up to rows_per_block.
 *
 * agcn_dist_set_graph takes the WHOLE degree-ordered square matrix on this
 * rank's device (every rank builds or loads the same one), keeps this rank's
 * block, renames its column ids to positions in the gathered operand, and
 * builds .block4 metadata and the plan for the block.  exchange_slices > 1
 * exchanges the operand in that many row slices and cuts the block's columns
 * the same way (agcn_spmm_tiled), so the product over a slice starts as soon
 * as the slice has arrived instead of after the whole all-gather.  With one
 * slice, column_ranges > 1 cuts the block's columns into that many equal
 * ranges of the gathered operand (for a gathered operand larger than L2:
 * agcn_spmm_tiled_suggest(rows_per_block, world * rows_per_block, local nnz,
 * dim) says how many); 1 = no tiling.
 *
 * Dense operands are "block rows": [rows_per_block x dim] per rank, row j =
 * local row j, padding rows zero.  agcn_dist_block_rows writes, for any rank,
 * the matrix row held at each local row (-1 = padding) -- what a caller needs
 * to scatter X into blocks and to put Y back into matrix order.
 *
 * agcn_dist_gather_begin starts the all-gather of this rank's block into one
 * of 4 slots on the context's communication stream, after the work already on
 * `stream`; agcn_dist_spmm_gathered makes `stream` wait for the slot (slice by
 * slice) and runs Y_block = act(A_block * X).  Products that do not depend on
 * each other can have their exchanges started together.  agcn_dist_spmm_step
 * is both calls on slot 0.  With world = 1 nothing is exchanged and the block
 * is read in place (it must stay valid until the product has run).  All calls
 * are asynchronous; every rank must issue the same sequence of exchanges, and a
 * slot's product must be enqueued before the slot's next exchange is begun.
 * ---------------------------------------------------------------------- */
#define AGCN_MAX_WORLD      64
#define AGCN_DIST_ID_BYTES 128
typedef struct agcn_dist agcn_dist;

int agcn_balanced_blocks(const int32_t *h_indptr, int64_t n_rows, int world,
                         int64_t *h_ranges, int64_t *rows_per_block);

/* id: AGCN_DIST_ID_BYTES bytes made by ONE rank and handed to all the others by the caller's own
 * means (a file, MPI, a torch.distributed broadcast) before they call agcn_dist_create. */
int agcn_dist_unique_id(void *id);
/* id == NULL with world > 1 creates a context WITHOUT a communicator: layout, block and local
 * product only, for callers that exchange the operand by their own means (or that run every
 * rank's block in one process); they use agcn_dist_spmm_on_gathered instead of the gather calls. */
int agcn_dist_create(agcn_dist **dist, int rank, int world, const void *id);
int agcn_dist_destroy(agcn_dist *dist);
int agcn_dist_set_graph(agcn_dist *dist, const int32_t *d_indptr, const int32_t *d_indices,
                        const float *d_vals, int64_t n_rows, int64_t nnz, int exchange_slices,
                        int column_ranges, void *stream);
int agcn_dist_info(const agcn_dist *dist, int64_t *rows_per_block, int64_t *local_rows,
                   int64_t *local_nnz, int64_t *n_blocks, int *exchange_slices,
                   int *launches_last_step);
int agcn_dist_block_rows(const agcn_dist *dist, int rank, int32_t *d_rows /* [rows_per_block] */,
                         void *stream);
int agcn_dist_gather_begin(agcn_dist *dist, int slot, const float *d_x_block, int dim, void *stream);
int agcn_dist_spmm_gathered(agcn_dist *dist, int slot, float *d_y_block, int dim, int activation,
                            void *stream);
int agcn_dist_spmm_step(agcn_dist *dist, const float *d_x_block, float *d_y_block, int dim,
                        int activation, void *stream);
/* makes `stream` wait for the whole exchange of a slot without multiplying (timing the exchange alone) */
int agcn_dist_wait_gathered(agcn_dist *dist, int slot, void *stream);
/* Y_block = act(A_block * X) on an operand the caller assembled itself: d_gathered is
 * [world * rows_per_block x dim], rank g's block rows at rows g * rows_per_block ... (with
 * exchange_slices > 1: slice c of every rank first, as agcn_dist_gather_begin lays it out). */
int agcn_dist_spmm_on_gathered(agcn_dist *dist, const float *d_gathered, float *d_y_block, int dim,
                               int activation, void *stream);
/* the gathered operand of a slot (valid after the exchange has completed), for inspection */
int agcn_dist_gathered(const agcn_dist *dist, int slot, const float **d_gathered, int64_t *n_rows);

/* ------------------------------------------------------------------------
 * Two-layer GCN forward  relu(A relu(A X W1) W2)  on the row blocks, 128
 * features: per layer Z = H * W (agcn_gemm_tf32_async on the owned rows), the
 * all-gather of Z, relu(A_block * Z) (the SpMM with its fused activation).
 * The reference stops at the SpMM (spmm_accel.cu:104-108); this is the workload
 * its operator exists for.  W1 / W2 are borrowed [128 x 128] device arrays.
 * run enqueues one forward on `stream` and returns; after synchronising that
 * stream, agcn_gcn2_forward_status reports a dense transform whose bounded wait
 * ran out (AGCN_ERR_CUDA) and, if ms6 is not NULL, six times in milliseconds:
 * per layer the transform, the wait for the exchange's first slice, the SpMM.
 * ---------------------------------------------------------------------- */
typedef struct agcn_gcn2 agcn_gcn2;

int agcn_gcn2_forward_create(agcn_gcn2 **fwd, agcn_dist *dist, const float *d_w1, const float *d_w2);
int agcn_gcn2_forward_run(agcn_gcn2 *fwd, const float *d_x_block, float *d_out_block, void *stream);
int agcn_gcn2_forward_status(agcn_gcn2 *fwd, float *ms6);
int agcn_gcn2_forward_destroy(agcn_gcn2 *fwd);

/* ------------------------------------------------------------------------
 * Measurement aid (not on the product path): the rate, in GB/s, at which this
 * GPU gathers whole rows of an L2-resident table with the access shape of the
 * SpMM (16-byte lanes, four rows in flight per lane, same residency and L2
 * policy, a chosen number of resident thread blocks per SM) -- the ceiling of a gather SpMM on graphs dense enough that X is
 * re-read from L2 rather than from HBM.  row_floats is 32, 64 or 128; table_rows
 * is a power of two.
 * ---------------------------------------------------------------------- */
int agcn_probe_gather_bandwidth(int64_t table_rows, int row_floats, int64_t total_rows, int iters,
                                int resident_blocks /* per SM; 0 = no limit, the SpMM keeps 5 */,
                                double *gb_per_s);

#ifdef __cplusplus
}
#endif
#endif /* ACCELGCN_H */
