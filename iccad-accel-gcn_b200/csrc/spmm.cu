// C-ABI entry points of the SpMM plug-in (replaces SPMM_ACCEL,
// spmm_accel.cu:104-139) and of the host-buffer call.
#include "host_common.h"
#include "internal.h"
#include "kernels/spmm_kernels.cuh"

#include <cstdlib>
#include <new>

namespace agcn {

int env_int(const char *name, int dflt)
{
    const char *v = getenv(name);
    return v != nullptr && *v ? atoi(v) : dflt;
}

void plan_free(agcn_spmm_plan *p)
{
    if (p == nullptr) return;
    cudaFree(p->unit_carry);
    cudaFree(p->carry_row);
    cudaFree(p->carry);
    cudaFree(p->zero_rows);
    cudaFree(p->x_pad);
    delete p;
}

int spmm_create(agcn_spmm_plan **out, const int *d_block4, int64_t n_blocks, const int *d_indices,
                       int64_t n_rows, int64_t n_cols, int64_t nnz, cudaStream_t s)
{
    AGCN_REQUIRE(out != nullptr, "agcn_spmm_create: null plan pointer");
    *out = nullptr;
    AGCN_REQUIRE(n_blocks >= 0 && (n_blocks == 0 || d_block4 != nullptr), "agcn_spmm_create: null block4");
    AGCN_REQUIRE(aligned16(d_block4), "agcn_spmm_create: block4 must be 16-byte aligned");
    AGCN_REQUIRE(n_rows > 0 && n_rows < (int64_t)INT32_MAX && n_cols > 0 && n_cols < (int64_t)INT32_MAX,
                 "agcn_spmm_create: n_rows / n_cols out of range");
    AGCN_REQUIRE(nnz >= 0 && nnz <= (int64_t)INT32_MAX, "agcn_spmm_create: nnz out of range");
    AGCN_REQUIRE(n_blocks < (int64_t)INT32_MAX, "agcn_spmm_create: too many blocks");

    const int4 *block4 = reinterpret_cast<const int4 *>(d_block4);
    const int64_t n_units = ceil_div(n_blocks, SPMM_WARPS);
    DeviceScratch scratch;
    AGCN_ALLOC(gap, scratch, int, n_blocks + 1);
    AGCN_ALLOC(gap_offset, scratch, int64_t, n_blocks + 1);
    AGCN_ALLOC(cnt, scratch, int, n_units);
    AGCN_ALLOC(slot_offset, scratch, int64_t, n_units);
    AGCN_ALLOC(tile_sums, scratch, int64_t, scan_tiles(n_blocks + 1));
    AGCN_ALLOC(d_res, scratch, int64_t, 3);    // [0] zero rows, [1] carry slots, [2] error bits (low int)
    AGCN_CUDA(cudaMemsetAsync(d_res, 0, 3 * sizeof(int64_t), s));
    int *d_err = reinterpret_cast<int *>(d_res + 2);

    AGCN_KERNEL(plan_check_kernel, (unsigned)ceil_div(n_blocks + 1, 256), 256, s, block4, n_blocks, n_rows, nnz, gap, d_err);
    AGCN_LAUNCH_CHECK("plan_check_kernel");
    if (d_indices != nullptr && nnz > 0) {
        int rc_cols = spmm_check_cols(d_indices, nnz, n_cols, d_err, s);
        if (rc_cols != AGCN_OK) return rc_cols;
    }
    int rc = exclusive_scan_i32_i64(gap, gap_offset, n_blocks + 1, tile_sums, d_res + 0, s);
    if (rc != AGCN_OK) return rc;
    if (n_units > 0) {
        AGCN_KERNEL(plan_count_carry_kernel, (unsigned)ceil_div(n_units, 256), 256, s, block4, n_blocks, n_units, cnt);
        AGCN_LAUNCH_CHECK("plan_count_carry_kernel");
        rc = exclusive_scan_i32_i64(cnt, slot_offset, n_units, tile_sums, d_res + 1, s);
        if (rc != AGCN_OK) return rc;
    }
    int64_t res[3] = {0, 0, 0};
    AGCN_CUDA(cudaMemcpyAsync(res, d_res, sizeof(res), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaStreamSynchronize(s));
    const int err = (int)(res[2] & 0xffffffff);
    if (err != 0) {
        set_error("agcn_spmm_create: invalid input:%s%s%s%s",
                  (err & SPMM_ERR_TUPLE) ? " malformed .block4 tuple;" : "",
                  (err & SPMM_ERR_ROW) ? " tuple rows out of range or not ascending;" : "",
                  (err & SPMM_ERR_LOC) ? " tuple nonzero range outside [0, nnz) or out of order;" : "",
                  (err & SPMM_ERR_COL) ? " column index outside [0, n_cols);" : "");
        return AGCN_ERR_RANGE;
    }

    agcn_spmm_plan *p = new (std::nothrow) agcn_spmm_plan;
    AGCN_REQUIRE(p != nullptr, "agcn_spmm_create: out of host memory");
    p->block4 = block4; p->n_blocks = n_blocks; p->n_units = n_units;
    p->n_rows = n_rows; p->n_cols = n_cols; p->nnz = nnz;
    p->n_zero = res[0]; p->n_carry = res[1];
    cudaError_t e = cudaSuccess;
    if (e == cudaSuccess && n_units > 0) e = cudaMalloc(&p->unit_carry, (size_t)n_units * sizeof(int2));
    if (e == cudaSuccess && p->n_carry > 0) e = cudaMalloc(&p->carry_row, (size_t)p->n_carry * sizeof(int));
    if (e == cudaSuccess && p->n_carry > 0) e = cudaMalloc(&p->carry, (size_t)p->n_carry * SPMM_PANEL * sizeof(float));
    if (e == cudaSuccess && p->n_zero > 0) e = cudaMalloc(&p->zero_rows, (size_t)p->n_zero * sizeof(int));
    if (e != cudaSuccess) {
        set_error("agcn_spmm_create: cudaMalloc of plan scratch: %s", cudaGetErrorString(e));
        plan_free(p);
        return AGCN_ERR_CUDA;
    }
    if (p->n_zero > 0)
        AGCN_KERNEL(plan_zero_rows_kernel, (unsigned)ceil_div(n_blocks + 1, 256), 256, s, block4, n_blocks, (const int *)gap,
                    (const int64_t *)gap_offset, p->zero_rows);
    if (n_units > 0)
        AGCN_KERNEL(plan_assign_carry_kernel, (unsigned)ceil_div(n_units, 256), 256, s, block4, n_blocks, n_units,
                    (const int64_t *)slot_offset, p->unit_carry, p->carry_row);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        set_error("agcn_spmm_create: plan kernels: %s", cudaGetErrorString(e));
        plan_free(p);
        return AGCN_ERR_CUDA;
    }
    {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&p->l2_bytes, cudaDevAttrL2CacheSize, dev);
        cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, dev);
        p->panel_override = env_int("AGCN_SPMM_PANEL", 0);
        p->pad_unaligned = env_int("AGCN_SPMM_PAD", 1);
        p->batch_override = env_int("AGCN_SPMM_BATCH", 0);
    }
    *out = p;
    return AGCN_OK;
}

// Column ids idx[0 .. count) against [0, n_cols): ORs SPMM_ERR_COL into *d_flag when one is outside.
int spmm_check_cols(const int *d_idx, int64_t count, int64_t n_cols, int *d_flag, cudaStream_t s)
{
    if (count <= 0) return AGCN_OK;
    const int64_t blocks = ceil_div(count, 256 * 16);
    AGCN_KERNEL(plan_check_cols_kernel, (unsigned)(blocks < 65535 ? blocks : 65535), 256, s, d_idx, count, n_cols, d_flag);
    AGCN_LAUNCH_CHECK("plan_check_cols_kernel");
    return AGCN_OK;
}

template <int S>
static void launch_units(const SpmmParams &prm, unsigned grid, bool small_launch, bool plain, int batch, cudaStream_t s)
{
    if (batch == 8) {          // experiment knob AGCN_SPMM_BATCH=8: 8 gathers in flight per lane at 3 thread blocks per SM
        if (plain) { auto k = spmm_units_kernel<S, 8, 3, true>; AGCN_KERNEL(k, grid, SPMM_THREADS, s, prm); }
        else { auto k = spmm_units_kernel<S, 8, 3, false>; AGCN_KERNEL(k, grid, SPMM_THREADS, s, prm); }
        return;
    }
    if (small_launch || batch == 16) {
        if (plain) { auto k = spmm_units_kernel<S, SPMM_SMALL_GATHER_BATCH, SPMM_SMALL_MIN_BLOCKS, true>; AGCN_KERNEL(k, grid, SPMM_THREADS, s, prm); }
        else { auto k = spmm_units_kernel<S, SPMM_SMALL_GATHER_BATCH, SPMM_SMALL_MIN_BLOCKS, false>; AGCN_KERNEL(k, grid, SPMM_THREADS, s, prm); }
    } else {
        if (plain) { auto k = spmm_units_kernel<S, SPMM_GATHER_BATCH, SPMM_MIN_BLOCKS, true>; AGCN_KERNEL(k, grid, SPMM_THREADS, s, prm); }
        else { auto k = spmm_units_kernel<S, SPMM_GATHER_BATCH, SPMM_MIN_BLOCKS, false>; AGCN_KERNEL(k, grid, SPMM_THREADS, s, prm); }
    }
}

static void launch_units_for_width(int width, bool vec, const SpmmParams &prm, unsigned grid, bool small_launch, bool plain,
                                   int batch, cudaStream_t s)
{
    if (!vec) launch_units<0>(prm, grid, small_launch, plain, batch, s);
    else if (width <= 16) launch_units<4>(prm, grid, small_launch, plain, batch, s);
    else if (width <= 32) launch_units<8>(prm, grid, small_launch, plain, batch, s);
    else if (width <= 64) launch_units<16>(prm, grid, small_launch, plain, batch, s);
    else launch_units<32>(prm, grid, small_launch, plain, batch, s);
}

// Rows of X that are not 16-byte aligned (dim % 4 != 0 with the reference's ld = dim, an odd
// stride or base) would force 4-byte gathers: 1.2-1.6x the time of the 16-byte path.  Instead X
// is copied once into plan-owned rows padded to a multiple of 4 floats (2 * n_cols * dim * 4
// bytes of streaming traffic against nnz * dim * 4 bytes of gather) and the 16-byte path runs
// on the copy; Y keeps the caller's layout and gets element-wise stores where it is unaligned.
// On return *x_use / *ldx_use name the operand to gather from and *x_vec says whether its rows
// are 16-byte aligned.
int spmm_prepare_x(agcn_spmm_plan *p, const float *d_x, int64_t ldx, int dim, cudaStream_t s,
                   const float **x_use, int64_t *ldx_use, bool *x_vec)
{
    const bool x_aligned = dim % 4 == 0 && ldx % 4 == 0 && aligned16(d_x);
    *x_use = d_x;
    *ldx_use = ldx;
    *x_vec = x_aligned;
    if (x_aligned || !p->pad_unaligned || p->nnz == 0) return AGCN_OK;
    const int ldp = (dim + 3) & ~3;
    const size_t need = (size_t)p->n_cols * ldp * sizeof(float);
    if (need > p->x_pad_bytes) {
        // growing the scratch synchronises the device once per plan and width; steady state allocates nothing
        if (p->x_pad != nullptr) AGCN_CUDA(cudaFree(p->x_pad));
        p->x_pad = nullptr; p->x_pad_bytes = 0;
        AGCN_CUDA(cudaMalloc(&p->x_pad, need));
        p->x_pad_bytes = need;
    }
    const int64_t quads = p->n_cols * (ldp >> 2);
    AGCN_KERNEL(spmm_pad_rows_kernel, (unsigned)ceil_div(quads, 256), 256, s, d_x, ldx, dim, p->x_pad, ldp, p->n_cols);
    AGCN_LAUNCH_CHECK("spmm_pad_rows_kernel");
    p->launches_last_run++;
    *x_use = p->x_pad;
    *ldx_use = ldp;
    *x_vec = true;
    return AGCN_OK;
}

int spmm_check_run_args(const agcn_spmm_plan *p, const int *d_indices, const float *d_vals, const float *d_x, int64_t ldx,
                        const float *d_y, int64_t ldy, int dim, int activation)
{
    AGCN_REQUIRE(activation == 0 || activation == 1, "agcn_spmm_run_act: activation must be AGCN_ACT_NONE or AGCN_ACT_RELU");
    AGCN_REQUIRE(p != nullptr, "agcn_spmm_run: null plan");
    AGCN_REQUIRE(d_x != nullptr && d_y != nullptr, "agcn_spmm_run: null X or Y");
    AGCN_REQUIRE(p->nnz == 0 || (d_indices != nullptr && d_vals != nullptr), "agcn_spmm_run: null indices or values");
    AGCN_REQUIRE(dim >= 1, "agcn_spmm_run: dim = %d", dim);
    AGCN_REQUIRE(ldx >= dim && ldy >= dim, "agcn_spmm_run: row stride smaller than dim");
    return AGCN_OK;
}

// One product on one set of tuples, X already prepared.  accumulate: Y += A * X (a later column
// range of a column-tiled product; rows no tuple covers then keep their value, and only get the
// activation).
int spmm_run_prepared(agcn_spmm_plan *p, const int *d_indices, const float *d_vals, const float *x_use, int64_t ldx_use,
                      bool x_vec, float *d_y, int64_t ldy, int dim, cudaStream_t s, int activation, int accumulate,
                      const SpmmLaunchPart &part)
{
    const int64_t unit0 = part.unit0, unit1 = part.unit1 < 0 ? p->n_units : part.unit1;
    AGCN_REQUIRE(unit0 >= 0 && unit0 <= unit1 && unit1 <= p->n_units, "agcn_spmm_run: unit range outside the plan");
    // rows no tuple covers: zero-filled -- or, when accumulating, left alone unless an activation is due
    const int64_t zero_blocks = !part.zero_fill || (accumulate && !activation) ? 0 : ceil_div(p->n_zero, SPMM_ZERO_ROWS_PER_BLOCK);
    const int64_t grid = (unit1 - unit0) + zero_blocks;
    AGCN_REQUIRE(grid < (int64_t)INT32_MAX, "agcn_spmm_run: grid too large");
    const bool small_launch = p->n_units <= (int64_t)SPMM_SMALL_MIN_BLOCKS * p->sm_count;

    // Column panels.  The gather re-reads a row of X once per nonzero of that column, so it runs
    // at L2 speed only while the X columns of a pass stay L2-resident.  When dim > 64 and the
    // operand is somewhat larger than what L2 keeps, two 64-column passes (each re-streaming the
    // 8 bytes per nonzero of A) beat one 128-column pass that spills to HBM (measured on B200:
    // 3.8 ms against 4.2-4.7 ms at N = 250 000, dim 128; 0.77 against 0.86 ms at N = 500 000).
    // When X is many times larger than L2 neither pass fits and one pass is as fast or faster
    // (6.3 against 6.5 ms at N = 5 000 000), so the split is limited to operands up to 4x L2.
    // Passes stay multiples of 32 columns so that every row segment is whole 128-byte lines.
    // AGCN_SPMM_PANEL (read when the plan is created) overrides the choice.  (A product whose A is
    // column-tiled -- agcn_spmm_tiled_* -- keeps its X slab in L2 by construction and never splits.)
    int panel = SPMM_PANEL;
    if (dim > 64 && dim % 32 == 0 && ldx_use % 32 == 0 && !accumulate && !p->never_split) {
        const int full = dim < SPMM_PANEL ? dim : SPMM_PANEL;
        const double x_bytes = (double)p->n_cols * full * 4.0;
        if (x_bytes > 0.75 * (double)p->l2_bytes && x_bytes <= 4.0 * (double)p->l2_bytes) panel = 64;
    }
    if (p->panel_override > 0) panel = p->panel_override;
    const int64_t cs0 = part.carry_s0, cs1 = part.carry_s1 < 0 ? p->n_carry : part.carry_s1;
    AGCN_REQUIRE(cs0 >= 0 && cs0 <= cs1 && cs1 <= p->n_carry, "agcn_spmm_run: carry slot range outside the plan");
    const bool whole = unit0 == 0 && unit1 == p->n_units && part.carry && cs0 == 0 && cs1 == p->n_carry;
    // A carry slot holds SPMM_PANEL floats and every column pass uses its own columns of it, so a
    // product of up to SPMM_PANEL columns can be issued in parts (unit launches now, carry kernel
    // later) whatever its passes are -- with the same passes, hence the same bits, as a whole run.
    if (!whole) AGCN_REQUIRE(dim <= SPMM_PANEL, "agcn_spmm_run: a product issued in unit ranges is limited to %d columns", SPMM_PANEL);
    AGCN_REQUIRE(panel >= 1 && panel <= SPMM_PANEL, "agcn_spmm_run: AGCN_SPMM_PANEL must be 1..%d", SPMM_PANEL);
    if (x_vec && panel % 4 != 0) panel = (panel + 3) & ~3;         // keep every panel's first column 16-byte aligned
    if (panel > SPMM_PANEL) panel = SPMM_PANEL;
    for (int col0 = 0; col0 < dim; col0 += panel) {
        const int width = dim - col0 < panel ? dim - col0 : panel;
        SpmmParams prm;
        prm.block4 = p->block4; prm.n_blocks = p->n_blocks;
        prm.n_units = unit1 - unit0; prm.unit_base = unit0; prm.abort_flag = part.abort_flag;
        prm.idx = d_indices; prm.val = d_vals;
        prm.x = x_use + col0; prm.ldx = ldx_use;
        prm.y = d_y + col0; prm.ldy = ldy;
        prm.unit_carry = p->unit_carry;
        prm.carry = (part.carry_buf != nullptr ? part.carry_buf : p->carry) + col0 % SPMM_PANEL;
        prm.zero_rows = p->zero_rows; prm.n_zero_rows = p->n_zero;
        prm.relu = activation;
        prm.accumulate = accumulate;
        const bool vec = x_vec && aligned16(prm.x);
        const bool y_vec = width % 4 == 0 && ldy % 4 == 0 && aligned16(prm.y);
        prm.y_vec = y_vec ? 1 : 0;
        prm.dim_store = width;
        prm.dim = vec ? (width + 3) & ~3 : width;       // columns gathered (the padded copy holds zeros past dim)
        const bool plain = !accumulate && (vec ? y_vec : true);
        if (grid > 0) {
            launch_units_for_width(prm.dim, vec, prm, (unsigned)grid, small_launch, plain, p->batch_override, s);
            AGCN_LAUNCH_CHECK("spmm_units_kernel");
            p->launches_last_run++;
        }
        if (cs1 > cs0 && part.carry) {
            const unsigned cgrid = (unsigned)ceil_div(cs1 - cs0, SPMM_WARPS);
            auto k = vec ? spmm_carry_kernel<true> : spmm_carry_kernel<false>;
            AGCN_KERNEL(k, cgrid, SPMM_THREADS, s, (const float *)prm.carry, (const int *)p->carry_row, cs0, cs1, prm.y, ldy,
                        prm.dim, activation, accumulate, prm.y_vec, prm.dim_store);
            AGCN_LAUNCH_CHECK("spmm_carry_kernel");
            p->launches_last_run++;
        }
    }
    return AGCN_OK;
}

int spmm_run(agcn_spmm_plan *p, const int *d_indices, const float *d_vals, const float *d_x, int64_t ldx,
             float *d_y, int64_t ldy, int dim, cudaStream_t s, int activation, int accumulate)
{
    int rc = spmm_check_run_args(p, d_indices, d_vals, d_x, ldx, d_y, ldy, dim, activation);
    if (rc != AGCN_OK) return rc;
    p->launches_last_run = 0;
    const float *x_use = nullptr;
    int64_t ldx_use = 0;
    bool x_vec = false;
    rc = spmm_prepare_x(p, d_x, ldx, dim, s, &x_use, &ldx_use, &x_vec);
    if (rc != AGCN_OK) return rc;
    return spmm_run_prepared(p, d_indices, d_vals, x_use, ldx_use, x_vec, d_y, ldy, dim, s, activation, accumulate, SpmmLaunchPart());
}

}  // namespace agcn

extern "C" int agcn_spmm_create(agcn_spmm_plan **plan, const int32_t *d_block4, int64_t n_blocks,
                                const int32_t *d_indices, int64_t n_rows, int64_t n_cols, int64_t nnz, void *stream)
{
    agcn::clear_error();
    return agcn::spmm_create(plan, d_block4, n_blocks, d_indices, n_rows, n_cols, nnz, static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_spmm_run(agcn_spmm_plan *plan, const int32_t *d_indices, const float *d_vals,
                             const float *d_x, int64_t ldx, float *d_y, int64_t ldy, int dim, void *stream)
{
    agcn::clear_error();
    return agcn::spmm_run(plan, d_indices, d_vals, d_x, ldx, d_y, ldy, dim, static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_spmm_run_act(agcn_spmm_plan *plan, const int32_t *d_indices, const float *d_vals,
                                 const float *d_x, int64_t ldx, float *d_y, int64_t ldy, int dim, int activation,
                                 void *stream)
{
    agcn::clear_error();
    return agcn::spmm_run(plan, d_indices, d_vals, d_x, ldx, d_y, ldy, dim, static_cast<cudaStream_t>(stream), activation);
}

extern "C" int agcn_spmm_destroy(agcn_spmm_plan *plan)
{
    agcn::clear_error();
    agcn::plan_free(plan);
    return AGCN_OK;
}

extern "C" int agcn_spmm_plan_info(const agcn_spmm_plan *plan, int64_t *n_units, int64_t *n_carry,
                                   int64_t *n_zero_rows, int *launches_last_run)
{
    agcn::clear_error();
    AGCN_REQUIRE(plan != nullptr, "agcn_spmm_plan_info: null plan");
    if (n_units) *n_units = plan->n_units;
    if (n_carry) *n_carry = plan->n_carry;
    if (n_zero_rows) *n_zero_rows = plan->n_zero;
    if (launches_last_run) *launches_last_run = plan->launches_last_run;
    return AGCN_OK;
}
