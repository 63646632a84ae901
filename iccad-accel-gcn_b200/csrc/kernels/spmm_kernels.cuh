// Block-level-partitioned CSR SpMM for sm_100a:  Y[n_rows x dim] = A * X,
// A given as the degree-ordered (idx, val) arrays plus `.block4` metadata
// (one tuple {degree, row_begin, loc_begin, info} per block of <= 384
// nonzeros; decode rules of spmm_accel.cu:18-34).
//
// Work decomposition.  A thread block ("unit") takes SPMM_WARPS consecutive
// tuples, one per warp.  A warp first stages its tuple's (col, val) slice --
// at most 384 pairs -- into shared memory with coalesced loads, then walks it.
// The columns of one dense row are covered by a "slot" of S lanes, each lane
// holding a float4 (the counterpart of the reference's combined warp,
// spmm_accel.cu:36-53, with 16-byte instead of 4-byte lanes); a warp therefore
// works on 32/S nonzeros at a time.  Rows of degree <= 32 are given one slot
// each, longer rows are split over the slots of the warp and folded with
// butterfly shuffles.  Accumulators live in registers.
//
// Heavy rows (degree > 384) span several tuples.  Their per-tuple partial sums
// meet in shared memory and are added in tuple order; a row that is contained
// in one unit is then stored directly.  A row that crosses a unit boundary
// leaves one partial per unit in a small "carry" array (at most two per unit),
// and spmm_carry_kernel adds those in unit order.  Every element of Y is thus
// written exactly once with a plain store, in a fixed order of additions: no
// atomics, no dependence on what Y held before, bit-identical from run to run.
// Rows no tuple covers (degree 0) are zero-filled by extra blocks of the same
// launch.
#pragma once
#include "primitives.cuh"
#include "ptx.cuh"

namespace agcn {

constexpr int SPMM_DEG_BOUND = 384;    // format constant of .block4 (spmm_accel.cu:11)
// tuples per unit, one per warp (4, 6 and 12 were measured within 2 % of 8; override to experiment)
#ifndef AGCN_SPMM_WARPS
#define AGCN_SPMM_WARPS 8
#endif
constexpr int SPMM_WARPS = AGCN_SPMM_WARPS;
constexpr int SPMM_THREADS = SPMM_WARPS * 32;
constexpr int SPMM_PANEL = 128;        // dense columns covered by one launch
constexpr int SPMM_ZERO_ROWS_PER_BLOCK = 64;
// Gathers a lane keeps in flight, and thread blocks per SM the register budget is capped for.
// Measured on B200: 4 in flight x 5 blocks (40 warps per SM, 48 registers) beats 8 x 3 by 10-20 %
// and 2 x 6 / 2 x 7 by up to 30 % -- the gather wants occupancy more than per-warp depth.
constexpr int SPMM_GATHER_BATCH = 4;
constexpr int SPMM_MIN_BLOCKS = 40 / SPMM_WARPS;      // 40 resident warps per SM
// Small launches (a few thread blocks per SM at most) cannot hide latency with occupancy: there each
// warp walks its tuple alone, so the variant used for them trades registers for a deeper batch.
constexpr int SPMM_SMALL_GATHER_BATCH = 16;
constexpr int SPMM_SMALL_MIN_BLOCKS = 16 / SPMM_WARPS;

struct SpmmParams {
    const int4 *block4;
    int64_t n_blocks;
    int64_t n_units;          // units of this launch (thread blocks beyond them zero-fill uncovered rows)
    int64_t unit_base;        // first unit of this launch: a product may be launched as several unit ranges
    const int *abort_flag;    // optional: a nonzero word makes every thread block return at once
    const int *idx;
    const float *val;
    const float *x;     // first column of the panel
    int64_t ldx;        // floats between consecutive rows of X
    float *y;
    int64_t ldy;
    int dim;            // columns in this panel, 1..SPMM_PANEL
    const int2 *unit_carry;   // per unit: carry slot of a row entering / leaving the unit, or -1
    float *carry;             // [n_carry][SPMM_PANEL]
    const int *zero_rows;     // rows no tuple covers
    int64_t n_zero_rows;
    int relu;                 // nonzero: Y = max(A * X, 0) (fused GCN activation)
    // The fields below are read only by the general (PLAIN = false) kernel flavour.
    int accumulate;           // nonzero: Y += A * X (later column ranges of a column-tiled product)
    int y_vec;                // nonzero: rows of Y are 16-byte aligned and dim_store % 4 == 0
    int dim_store;            // columns of Y written (dim rounded up to 4 is what is gathered)
};

struct TupleView {
    int row0, loc, n_rows, row_nz;
    bool valid, small;
};

__device__ __forceinline__ TupleView decode_tuple(const int4 *__restrict__ block4, int64_t e, int64_t n_blocks)
{
    TupleView t;
    t.valid = e < n_blocks;
    const int4 b = t.valid ? __ldg(block4 + e) : make_int4(0, 0, 0, 0);
    t.small = b.x <= SPMM_DEG_BOUND;
    t.row0 = b.y;
    t.loc = b.z;
    t.n_rows = t.small ? (b.w & 0xffff) : 1;
    t.row_nz = t.small ? b.x : b.w;
    if (!t.valid) { t.n_rows = 0; t.row_nz = 0; }
    return t;
}

// ---------------------------------------------------------------------------
// gather-accumulate over the staged pairs  first, first+step, ... < count
// ---------------------------------------------------------------------------
__device__ __forceinline__ float4 relu4(const float4 &v, int on)
{
    return on ? make_float4(fmaxf(v.x, 0.f), fmaxf(v.y, 0.f), fmaxf(v.z, 0.f), fmaxf(v.w, 0.f)) : v;
}
__device__ __forceinline__ float relu1(float v, int on) { return on ? fmaxf(v, 0.f) : v; }

// Writes columns col .. col+3 of one result row.  PLAIN: one 16-byte store.  Otherwise the row may
// be unaligned or end inside the four columns (dim not a multiple of 4: element-wise stores), and
// the product may be added to what the row holds (column-tiled products).
template <bool PLAIN>
__device__ __forceinline__ void emit_row4(const SpmmParams &p, float *yr, int col, float4 v, int act, uint64_t policy)
{
    if (PLAIN) {
        st_y4(yr + col, relu4(v, act), policy);
    } else if (p.y_vec) {
        if (p.accumulate) {
            const float4 o = *reinterpret_cast<const float4 *>(yr + col);
            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
        st_y4(yr + col, relu4(v, act), policy);
    } else {
        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; k++)
            if (col + k < p.dim_store) st_y1(yr + col + k, relu1(p.accumulate ? e[k] + yr[col + k] : e[k], act), policy);
    }
}
template <bool PLAIN>
__device__ __forceinline__ void emit_row1(const SpmmParams &p, float *y, float v, int act, uint64_t policy)
{
    st_y1(y, relu1(!PLAIN && p.accumulate ? v + *y : v, act), policy);
}

__device__ __forceinline__ void fma4(float4 &acc, float a, const float4 &v)
{
    acc.x = fmaf(a, v.x, acc.x);
    acc.y = fmaf(a, v.y, acc.y);
    acc.z = fmaf(a, v.z, acc.z);
    acc.w = fmaf(a, v.w, acc.w);
}

// UNROLL independent 16-byte loads are issued per lane before the first FMA needs one.
template <int UNROLL>
__device__ __forceinline__ float4 gather_vec4(const int2 *pairs, int count, int first, int step,
                                              const float *__restrict__ x, int64_t ldx, bool active, uint64_t keep)
{
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!active) return acc;
    int i = first;
    for (; i + (UNROLL - 1) * step < count; i += UNROLL * step) {
        int2 p[UNROLL];
        float4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) p[u] = pairs[i + u * step];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) v[u] = ld_x4(x + (int64_t)p[u].x * ldx, keep);
#pragma unroll
        for (int u = 0; u < UNROLL; u++) fma4(acc, __int_as_float(p[u].y), v[u]);
    }
    if (i < count) {
        // tail: the same batch with the loads past the end switched off
        int2 p[UNROLL - 1];
        float4 v[UNROLL - 1];
#pragma unroll
        for (int u = 0; u < UNROLL - 1; u++) {
            const bool live = i + u * step < count;
            p[u] = live ? pairs[i + u * step] : make_int2(0, 0);
            v[u] = live ? ld_x4(x + (int64_t)p[u].x * ldx, keep) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < UNROLL - 1; u++)
            if (i + u * step < count) fma4(acc, __int_as_float(p[u].y), v[u]);
    }
    return acc;
}

constexpr int SPMM_SCALAR_COLS = SPMM_PANEL / 32;   // columns per lane in scalar mode

// Scalar mode: lane l owns columns l, l+32, ... (K = ceil(dim / 32) of them), every load instruction
// of the warp reads 128 contiguous bytes of one X row.  Nonzeros are taken in batches so that about
// 8 loads per lane are in flight, as in the float4 mode.
template <int K>
__device__ __forceinline__ void gather_strided(const int2 *pairs, int count, const float *__restrict__ x,
                                               int64_t ldx, int dim, float (&acc)[SPMM_SCALAR_COLS], uint64_t keep)
{
    constexpr int U = K <= 2 ? 4 : 2;        // nonzeros per batch
    const int lane = lane_id();
    bool live[K];
#pragma unroll
    for (int k = 0; k < K; k++) live[k] = lane + 32 * k < dim;
#pragma unroll
    for (int k = 0; k < SPMM_SCALAR_COLS; k++) acc[k] = 0.f;
    int i = 0;
    for (; i + U <= count; i += U) {
        int2 p[U];
        float v[U][K];
#pragma unroll
        for (int u = 0; u < U; u++) p[u] = pairs[i + u];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const float *xr = x + (int64_t)p[u].x * ldx + lane;
#pragma unroll
            for (int k = 0; k < K; k++) v[u][k] = live[k] ? ld_x1(xr + 32 * k, keep) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int k = 0; k < K; k++) acc[k] = fmaf(__int_as_float(p[u].y), v[u][k], acc[k]);
    }
    for (; i < count; i++) {
        const int2 p0 = pairs[i];
        const float *xr = x + (int64_t)p0.x * ldx + lane;
#pragma unroll
        for (int k = 0; k < K; k++)
            if (live[k]) acc[k] = fmaf(__int_as_float(p0.y), ld_x1(xr + 32 * k, keep), acc[k]);
    }
}

__device__ __forceinline__ void gather_scalar(const int2 *pairs, int count, const float *__restrict__ x,
                                              int64_t ldx, int dim, float (&acc)[SPMM_SCALAR_COLS], uint64_t keep)
{
    switch ((dim + 31) >> 5) {            // uniform over the launch
    case 1: gather_strided<1>(pairs, count, x, ldx, dim, acc, keep); break;
    case 2: gather_strided<2>(pairs, count, x, ldx, dim, acc, keep); break;
    case 3: gather_strided<3>(pairs, count, x, ldx, dim, acc, keep); break;
    default: gather_strided<4>(pairs, count, x, ldx, dim, acc, keep); break;
    }
}

// ---------------------------------------------------------------------------
// main kernel.  S = lanes per slot in float4 mode (4, 8, 16 or 32; needs
// dim % 4 == 0, dim <= 4*S and 16-byte aligned rows); S = 0 is the scalar
// mode for every other dim (lane l owns columns l, l+32, l+64, l+96).
// ---------------------------------------------------------------------------
template <int S, int BATCH, int MIN_BLOCKS, bool PLAIN>
__global__ void __launch_bounds__(SPMM_THREADS, MIN_BLOCKS)
spmm_units_kernel(const SpmmParams p)
{
    __shared__ int2 s_pair[SPMM_WARPS][SPMM_DEG_BOUND];
    __shared__ __align__(16) float s_part[SPMM_WARPS][SPMM_PANEL];
    __shared__ int s_row[SPMM_WARPS];
    __shared__ int s_big[SPMM_WARPS];

    constexpr bool VEC = S > 0;
    constexpr int LANES = VEC ? S : 32;
    constexpr int NS = 32 / LANES;          // nonzeros a warp works on at a time
    const int w = warp_id(), lane = lane_id();
    const int slot = lane / LANES, sl = lane % LANES;
    const int col = VEC ? sl * 4 : sl;
    const bool active = col < p.dim;
    const L2Policies pol = make_l2_policies();

    if (p.abort_flag != nullptr && *p.abort_flag != 0) return;     // input rejected by a check earlier in the stream
    if ((int64_t)blockIdx.x >= p.n_units) {
        // zero-fill rows that no tuple covers
        // (when accumulating, these rows keep their value and only the activation is applied)
        const int64_t zb = ((int64_t)blockIdx.x - p.n_units) * SPMM_ZERO_ROWS_PER_BLOCK;
        for (int k = w * NS + slot; k < SPMM_ZERO_ROWS_PER_BLOCK; k += SPMM_WARPS * NS) {
            if (zb + k >= p.n_zero_rows) break;
            float *yr = p.y + (int64_t)p.zero_rows[zb + k] * p.ldy;
            if (VEC) {
                if (active) emit_row4<PLAIN>(p, yr, col, make_float4(0.f, 0.f, 0.f, 0.f), p.relu, pol.stream);
            } else {
                for (int c = lane; c < p.dim; c += 32) emit_row1<PLAIN>(p, yr + c, 0.f, p.relu, pol.stream);
            }
        }
        return;
    }

    const int64_t unit = p.unit_base + blockIdx.x;
    const int64_t e = unit * SPMM_WARPS + w;
    const TupleView t = decode_tuple(p.block4, e, p.n_blocks);
    const int total = t.n_rows * t.row_nz;

    // stage the tuple's (col, val) slice
    {
        const int *__restrict__ gi = p.idx + t.loc;
        const float *__restrict__ gv = p.val + t.loc;
#pragma unroll 4
        for (int k = lane; k < total; k += 32)
            s_pair[w][k] = make_int2(ld_a(gi + k, pol.stream), __float_as_int(ld_a(gv + k, pol.stream)));
    }
    __syncwarp();

    const bool big = t.valid && !t.small;
    const int2 *pairs = s_pair[w];

    if (VEC) {
        const float *xc = p.x + col;
        if (t.small && NS > 1 && t.row_nz <= 32) {
            // one slot per row
            for (int r = slot; r < t.n_rows; r += NS) {
                const float4 acc = gather_vec4<BATCH>(pairs + r * t.row_nz, t.row_nz, 0, 1, xc, p.ldx, active, pol.keep);
                if (active) emit_row4<PLAIN>(p, p.y + (int64_t)(t.row0 + r) * p.ldy, col, acc, p.relu, pol.stream);
            }
        } else {
            // the slots of the warp share each row
            for (int r = 0; r < t.n_rows; r++) {
                float4 acc = gather_vec4<BATCH>(pairs + r * t.row_nz, t.row_nz, slot, NS, xc, p.ldx, active, pol.keep);
#pragma unroll
                for (int off = LANES; off < 32; off <<= 1) {
                    acc.x += __shfl_xor_sync(FULL_MASK, acc.x, off);
                    acc.y += __shfl_xor_sync(FULL_MASK, acc.y, off);
                    acc.z += __shfl_xor_sync(FULL_MASK, acc.z, off);
                    acc.w += __shfl_xor_sync(FULL_MASK, acc.w, off);
                }
                if (slot == 0 && active) {
                    if (t.small) emit_row4<PLAIN>(p, p.y + (int64_t)(t.row0 + r) * p.ldy, col, acc, p.relu, pol.stream);
                    else *reinterpret_cast<float4 *>(&s_part[w][col]) = acc;
                }
            }
        }
    } else {
        for (int r = 0; r < t.n_rows; r++) {
            float acc[SPMM_SCALAR_COLS];
            gather_scalar(pairs + r * t.row_nz, t.row_nz, p.x, p.ldx, p.dim, acc, pol.keep);
#pragma unroll
            for (int k = 0; k < SPMM_SCALAR_COLS; k++) {
                const int c = lane + 32 * k;
                if (c < p.dim) {
                    if (t.small) emit_row1<PLAIN>(p, p.y + (int64_t)(t.row0 + r) * p.ldy + c, acc[k], p.relu, pol.stream);
                    else s_part[w][c] = acc[k];
                }
            }
        }
    }

    // heavy rows: add the per-tuple partials of a row in tuple order
    if (lane == 0) { s_row[w] = t.row0; s_big[w] = big ? 1 : 0; }
    __syncthreads();
    if (!big) return;
    if (w > 0 && s_big[w - 1] && s_row[w - 1] == t.row0) return;   // not the first tuple of its row here
    int w_end = w + 1;
    while (w_end < SPMM_WARPS && s_big[w_end] && s_row[w_end] == t.row0) w_end++;
    const int64_t left = p.n_blocks - unit * SPMM_WARPS;
    const int w_last = left < SPMM_WARPS ? (int)left - 1 : SPMM_WARPS - 1;
    const int2 uc = __ldg(p.unit_carry + unit);
    const bool enters = w == 0 && uc.x >= 0;            // the row began in an earlier unit
    const bool leaves = w_end - 1 == w_last && uc.y >= 0;   // the row goes on in the next unit
    const bool partial = enters || leaves;     // the row is finished by spmm_carry_kernel
    float *dst = partial ? p.carry + (int64_t)(enters ? uc.x : uc.y) * SPMM_PANEL : p.y + (int64_t)t.row0 * p.ldy;
    const int act = partial ? 0 : p.relu;
    if (VEC) {
        if (slot == 0 && active) {
            float4 sum = *reinterpret_cast<const float4 *>(&s_part[w][col]);
            for (int ww = w + 1; ww < w_end; ww++) {
                const float4 v = *reinterpret_cast<const float4 *>(&s_part[ww][col]);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            if (partial) *reinterpret_cast<float4 *>(dst + col) = sum;      // carry slots are aligned and private
            else emit_row4<PLAIN>(p, dst, col, sum, act, pol.stream);
        }
    } else {
        for (int c = lane; c < p.dim; c += 32) {
            float sum = s_part[w][c];
            for (int ww = w + 1; ww < w_end; ww++) sum += s_part[ww][c];
            if (partial) dst[c] = sum;
            else emit_row1<PLAIN>(p, dst + c, sum, act, pol.stream);
        }
    }
}

// Adds the carried partials of every row that crosses unit boundaries, in
// unit order, and stores the row.  One warp per carry slot; the warp of the
// first slot of a row does the work.  The launch covers slots [s0, s1), a range
// that begins and ends between rows (all slots by default; a product issued in
// unit ranges finishes the rows of each range as soon as its units have run).
template <bool VEC>
__global__ void __launch_bounds__(SPMM_THREADS)
spmm_carry_kernel(const float *__restrict__ carry, const int *__restrict__ carry_row, int64_t s0, int64_t s1,
                  float *y, int64_t ldy, int dim, int relu, int accumulate, int y_vec, int dim_store)
{
    const int64_t s = s0 + (int64_t)blockIdx.x * SPMM_WARPS + warp_id();
    if (s >= s1) return;
    const int row = carry_row[s];
    if (s > s0 && carry_row[s - 1] == row) return;
    int64_t s_end = s + 1;
    while (s_end < s1 && carry_row[s_end] == row) s_end++;
    const int lane = lane_id();
    if (VEC) {
        const int col = lane * 4;
        if (col < dim) {
            float4 sum = *reinterpret_cast<const float4 *>(carry + s * SPMM_PANEL + col);
            for (int64_t q = s + 1; q < s_end; q++) {
                const float4 v = *reinterpret_cast<const float4 *>(carry + q * SPMM_PANEL + col);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            float *yr = y + (int64_t)row * ldy;
            if (y_vec) {
                if (accumulate) {
                    const float4 o = *reinterpret_cast<const float4 *>(yr + col);
                    sum.x += o.x; sum.y += o.y; sum.z += o.z; sum.w += o.w;
                }
                *reinterpret_cast<float4 *>(yr + col) = relu4(sum, relu);
            } else {
                const float e[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                for (int k = 0; k < 4; k++)
                    if (col + k < dim_store) yr[col + k] = relu1(accumulate ? e[k] + yr[col + k] : e[k], relu);
            }
        }
    } else {
        for (int c = lane; c < dim; c += 32) {
            float sum = carry[s * SPMM_PANEL + c];
            for (int64_t q = s + 1; q < s_end; q++) sum += carry[q * SPMM_PANEL + c];
            float *ye = y + (int64_t)row * ldy + c;
            *ye = relu1(accumulate ? sum + *ye : sum, relu);
        }
    }
}

// X[n_rows x dim] with row stride ldx  ->  XP[n_rows x ldp], ldp = dim rounded up to 4, tail zero:
// the 16-byte-aligned copy of a dense operand whose rows are not (dim % 4 != 0 or an unaligned base).
// One thread per 16 bytes written.
__global__ void __launch_bounds__(256)
spmm_pad_rows_kernel(const float *__restrict__ x, int64_t ldx, int dim, float *__restrict__ xp, int ldp, int64_t n_rows)
{
    const int quads = ldp >> 2;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * quads) return;
    const int64_t row = i / quads;
    const int c = (int)(i - row * quads) * 4;
    const float *src = x + row * ldx + c;
    float4 v;
    v.x = c + 0 < dim ? __ldg(src + 0) : 0.f;
    v.y = c + 1 < dim ? __ldg(src + 1) : 0.f;
    v.z = c + 2 < dim ? __ldg(src + 2) : 0.f;
    v.w = c + 3 < dim ? __ldg(src + 3) : 0.f;
    *reinterpret_cast<float4 *>(xp + row * ldp + c) = v;
}

// ---------------------------------------------------------------------------
// plan: built once per `.block4` array
// ---------------------------------------------------------------------------
constexpr int SPMM_ERR_TUPLE = 1;     // malformed tuple (degree, row count or chunk length)
constexpr int SPMM_ERR_ROW = 2;       // rows out of range, overlapping or not ascending
constexpr int SPMM_ERR_LOC = 4;       // nonzero range outside [0, nnz)
constexpr int SPMM_ERR_COL = 8;       // column index outside [0, n_cols)

__device__ __forceinline__ bool tuple_is_big(const int4 &b) { return b.x > SPMM_DEG_BOUND; }
__device__ __forceinline__ int tuple_rows(const int4 &b) { return tuple_is_big(b) ? 1 : (b.w & 0xffff); }

// Checks every tuple, and counts the rows that lie between tuple e-1 and
// tuple e (gap[e]; gap[n_blocks] = rows after the last tuple).
__global__ void __launch_bounds__(256)
plan_check_kernel(const int4 *__restrict__ block4, int64_t n_blocks, int64_t n_rows, int64_t nnz,
                  int *__restrict__ gap, int *__restrict__ err_flag)
{
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e > n_blocks) return;
    int err = 0;
    int64_t prev_end = 0;       // first row not covered by tuples before e
    int64_t prev_loc_end = 0;   // first nonzero not covered by tuples before e
    if (e > 0) {
        const int4 a = block4[e - 1];
        prev_end = (int64_t)a.y + tuple_rows(a);
        prev_loc_end = (int64_t)a.z + (tuple_is_big(a) ? (int64_t)a.w : (int64_t)tuple_rows(a) * a.x);
    }
    if (e == n_blocks) {
        gap[e] = prev_end <= n_rows ? (int)(n_rows - prev_end) : 0;
        return;
    }
    const int4 b = block4[e];
    const bool big = tuple_is_big(b);
    const int rows = tuple_rows(b);
    const int64_t nz = big ? (int64_t)b.w : (int64_t)rows * b.x;
    if (b.x < 1 || rows < 1 || nz < 1 || nz > SPMM_DEG_BOUND) err |= SPMM_ERR_TUPLE;
    // tuples take their nonzeros in order and without overlap (what lets A be uploaded and multiplied
    // range by range: a tuple never reaches into a range that has not arrived)
    if (b.z < 0 || (int64_t)b.z + nz > nnz || (int64_t)b.z < prev_loc_end) err |= SPMM_ERR_LOC;
    int64_t g = (int64_t)b.y - prev_end;
    if (big && e > 0) {
        // a later chunk of the same heavy row repeats its row id
        const int4 a = block4[e - 1];
        if (tuple_is_big(a) && a.y == b.y) g = 0;
    }
    if (b.y < 0 || (int64_t)b.y + rows > n_rows || g < 0) { err |= SPMM_ERR_ROW; g = 0; }
    gap[e] = (int)g;
    if (err) atomicOr(err_flag, err);
}

__global__ void __launch_bounds__(256)
plan_check_cols_kernel(const int *__restrict__ idx, int64_t nnz, int64_t n_cols, int *__restrict__ err_flag)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    bool bad = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nnz; i += stride) {
        const int c = idx[i];
        bad |= c < 0 || c >= n_cols;
    }
    if (bad) atomicOr(err_flag, SPMM_ERR_COL);
}

// zero_rows[gap_offset[e] ...] = the rows of gap e
__global__ void __launch_bounds__(256)
plan_zero_rows_kernel(const int4 *__restrict__ block4, int64_t n_blocks, const int *__restrict__ gap,
                      const int64_t *__restrict__ gap_offset, int *__restrict__ zero_rows)
{
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e > n_blocks) return;
    const int g = gap[e];
    if (g == 0) return;
    int64_t prev_end = 0;
    if (e > 0) {
        const int4 a = block4[e - 1];
        prev_end = (int64_t)a.y + tuple_rows(a);
    }
    int *dst = zero_rows + gap_offset[e];
    for (int k = 0; k < g; k++) dst[k] = (int)(prev_end + k);
}

// Does a heavy row enter unit u from the left / leave it to the right?
__device__ __forceinline__ void unit_crossings(const int4 *__restrict__ block4, int64_t n_blocks, int64_t u,
                                               bool &enters, bool &leaves, bool &same_row, int &row_in, int &row_out)
{
    const int64_t e0 = u * SPMM_WARPS;
    const int64_t e1 = e0 + SPMM_WARPS < n_blocks ? e0 + SPMM_WARPS : n_blocks;   // one past the unit
    const int4 first = block4[e0], last = block4[e1 - 1];
    enters = false; leaves = false;
    if (e0 > 0 && tuple_is_big(first)) {
        const int4 a = block4[e0 - 1];
        enters = tuple_is_big(a) && a.y == first.y;
    }
    if (e1 < n_blocks && tuple_is_big(last)) {
        const int4 c = block4[e1];
        leaves = tuple_is_big(c) && c.y == last.y;
    }
    row_in = first.y; row_out = last.y;
    same_row = enters && leaves && first.y == last.y;
}

__global__ void __launch_bounds__(256)
plan_count_carry_kernel(const int4 *__restrict__ block4, int64_t n_blocks, int64_t n_units, int *__restrict__ count)
{
    const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= n_units) return;
    bool en, lv, same; int ri, ro;
    unit_crossings(block4, n_blocks, u, en, lv, same, ri, ro);
    count[u] = (en ? 1 : 0) + (lv ? 1 : 0) - (same ? 1 : 0);
}

__global__ void __launch_bounds__(256)
plan_assign_carry_kernel(const int4 *__restrict__ block4, int64_t n_blocks, int64_t n_units,
                         const int64_t *__restrict__ slot_offset, int2 *__restrict__ unit_carry,
                         int *__restrict__ carry_row)
{
    const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= n_units) return;
    bool en, lv, same; int ri, ro;
    unit_crossings(block4, n_blocks, u, en, lv, same, ri, ro);
    const int s = (int)slot_offset[u];
    int2 uc = make_int2(-1, -1);
    if (en) { uc.x = s; carry_row[s] = ri; }
    if (lv) {
        uc.y = same ? s : s + (en ? 1 : 0);
        if (!same) carry_row[uc.y] = ro;
    }
    unit_carry[u] = uc;
}

}  // namespace agcn
