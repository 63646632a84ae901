// Host-buffer SpMM: the plug-in for a harness whose arrays live in host memory (the split
// follows SPMM_BASE: constructor = graph, run(dim) = one product; spmm_base.h:9-20,
// spmm_accel.cu:104-139), pipelined over three streams.
//
// What crosses PCIe is fixed by the call (the graph, X per product up; Y per product down), so
// the work is to keep both copy engines and the SMs busy at once:
//  - uploads, kernels and downloads run on three streams chained by events;
//  - a product is launched as several unit ranges (a unit = 8 consecutive tuples); each range is
//    followed by the carry kernel over the carry slots of the rows it completes, and those rows are
//    downloaded while the next range computes;
//  - when the graph itself is part of the call (agcn_spmm_host_batch), column ids and values are
//    uploaded in the same ranges and every range is multiplied -- for all products -- as soon as
//    it has arrived, so the kernels and the downloads hide under the upload of A.
// One cudaMemcpyAsync per copy; pinned host memory gives full overlap (pageable memory works,
// staged by the driver).
#include "host_common.h"
#include "internal.h"

#include <algorithm>
#include <chrono>
#include <new>
#include <vector>

namespace agcn {
constexpr int HOST_SPMM_WARPS = 8;                    // tuples per unit (SPMM_WARPS of the kernels)
constexpr int HOST_SPMM_PANEL = 128;                  // widest product that can be issued in unit ranges
}

struct agcn_host_ctx {
    cudaStream_t s_up = nullptr, s_run = nullptr, s_down = nullptr;
    void *graph[3] = {nullptr, nullptr, nullptr};     // block4, idx, val
    size_t graph_cap[3] = {0, 0, 0};
    std::vector<void *> xbuf, ybuf, cbuf;             // per product of a batch: X, Y, carry scratch
    std::vector<size_t> xcap, ycap, ccap;
    agcn_spmm_plan *plan = nullptr;                   // of the graph set last
    int64_t n_rows = 0, n_cols = 0, nnz = 0, n_blocks = 0;
    // unit ranges a product is issued in, with the first row / first nonzero of each boundary
    std::vector<int64_t> part_unit, part_row, part_loc;
    std::vector<int64_t> part_slot;                   // carry slots [part_slot[k], part_slot[k+1]) finish the rows of range k
    std::vector<int2> h_unit_carry;                   // host copies of the plan's carry bookkeeping
    std::vector<int> h_carry_row;
    int *d_abort = nullptr;                           // device word: set when a column id is out of range
    std::vector<cudaEvent_t> events;
    size_t events_used = 0;
    // timing of the last agcn_spmm_host_batch call (agcn_host_last_timing)
    cudaEvent_t t_up0 = nullptr, t_up1 = nullptr, t_run0 = nullptr, t_run1 = nullptr, t_down1 = nullptr;
    float host_plan_ms = 0.f, host_enqueue_ms = 0.f;
    bool timed = false;
};

namespace agcn {

static int ctx_event(agcn_host_ctx *c, cudaEvent_t *out)
{
    if (c->events_used == c->events.size()) {
        cudaEvent_t e = nullptr;
        AGCN_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        c->events.push_back(e);
    }
    *out = c->events[c->events_used++];
    return AGCN_OK;
}

// `from` -> event -> `to`: everything enqueued on `to` afterwards runs after what `from` holds now
static int ctx_chain(agcn_host_ctx *c, cudaStream_t from, cudaStream_t to)
{
    cudaEvent_t e = nullptr;
    int rc = ctx_event(c, &e);
    if (rc != AGCN_OK) return rc;
    AGCN_CUDA(cudaEventRecord(e, from));
    AGCN_CUDA(cudaStreamWaitEvent(to, e, 0));
    return AGCN_OK;
}

static int reserve(void **buf, size_t *cap, size_t bytes)
{
    if (bytes <= *cap) return AGCN_OK;
    if (*buf != nullptr) AGCN_CUDA(cudaFree(*buf));
    *buf = nullptr; *cap = 0;
    AGCN_CUDA(cudaMalloc(buf, bytes));
    *cap = bytes;
    return AGCN_OK;
}

static int ctx_sync(agcn_host_ctx *c)
{
    cudaError_t e1 = cudaStreamSynchronize(c->s_up), e2 = cudaStreamSynchronize(c->s_run), e3 = cudaStreamSynchronize(c->s_down);
    c->events_used = 0;
    const cudaError_t e = e1 != cudaSuccess ? e1 : e2 != cudaSuccess ? e2 : e3;
    if (e != cudaSuccess) {
        set_error("agcn_host_spmm: %s", cudaGetErrorString(e));
        return AGCN_ERR_CUDA;
    }
    return AGCN_OK;
}

// Cuts the tuple list into about `want_parts` unit ranges of equal nonzero count, reading the
// caller's host copy of .block4 (tuples tile [0, nnz) in order, so loc_begin is monotone).
static void plan_part_cuts(agcn_host_ctx *c, const int *h_block4, int want_parts)
{
    const int64_t n_units = ceil_div(c->n_blocks, HOST_SPMM_WARPS);
    c->part_unit.assign(1, 0);
    c->part_row.assign(1, 0);
    c->part_loc.assign(1, 0);
    if (want_parts < 1) want_parts = 1;
    for (int k = 1; k < want_parts && n_units > 0; k++) {
        const int64_t target = c->nnz * k / want_parts;
        // first unit whose first tuple starts at or after `target`
        int64_t lo = c->part_unit.back(), hi = n_units;
        while (lo < hi) {
            const int64_t mid = lo + (hi - lo) / 2;
            if ((int64_t)h_block4[4 * mid * HOST_SPMM_WARPS + 2] < target) lo = mid + 1; else hi = mid;
        }
        if (lo <= c->part_unit.back() || lo >= n_units) continue;
        // the tuples have not been validated yet when this runs ahead of the plan: a cut is only
        // taken where it keeps rows and nonzero offsets inside the arrays and in order
        const int64_t row = h_block4[4 * lo * HOST_SPMM_WARPS + 1], loc = h_block4[4 * lo * HOST_SPMM_WARPS + 2];
        if (loc <= c->part_loc.back() || loc >= c->nnz || row < c->part_row.back() || row > c->n_rows) continue;
        c->part_unit.push_back(lo);
        c->part_row.push_back(row);
        c->part_loc.push_back(loc);
    }
    c->part_unit.push_back(n_units);
    c->part_row.push_back(c->n_rows);
    c->part_loc.push_back(c->nnz);
}

// The carry slots of every unit range (needs the plan's bookkeeping: build_plan).
static void plan_part_slots(agcn_host_ctx *c)
{
    const int64_t n_units = ceil_div(c->n_blocks, HOST_SPMM_WARPS);
    // Carry slots are handed out in unit order (a slot for the row entering a unit from the left,
    // one for the row leaving it to the right).  The rows a unit range completes own the slots up
    // to the first slot of the row that runs on into the next range, or -- if none does -- up to the
    // first slot of the next range's first unit.
    const int n_parts = (int)c->part_unit.size() - 1;
    const int64_t n_carry = (int64_t)c->h_carry_row.size();
    c->part_slot.assign(n_parts + 1, n_carry);
    c->part_slot[0] = 0;
    int64_t next_slot = 0;                // slots handed out to the units before u
    int k = 1;
    for (int64_t u = 0; u < n_units && k < n_parts; u++) {
        const int2 uc = c->h_unit_carry[u];
        if (u == c->part_unit[k]) {
            int64_t first = next_slot;
            if (uc.x >= 0) {              // a row enters this unit from the previous range: back to its first slot
                first = uc.x;
                while (first > 0 && c->h_carry_row[first - 1] == c->h_carry_row[uc.x]) first--;
            }
            c->part_slot[k++] = first;
        }
        if (uc.x >= 0 && uc.x >= next_slot) next_slot = uc.x + 1;
        if (uc.y >= 0 && uc.y >= next_slot) next_slot = uc.y + 1;
    }
}

static void plan_parts(agcn_host_ctx *c, const int *h_block4, int want_parts)
{
    plan_part_cuts(c, h_block4, want_parts);
    plan_part_slots(c);
}

static int check_graph_args(agcn_host_ctx *ctx, const int *h_block4, int64_t n_blocks, const int *h_indices,
                            const float *h_vals, int64_t n_rows, int64_t n_cols, int64_t nnz)
{
    AGCN_REQUIRE(ctx != nullptr, "agcn_host_set_graph: null context");
    AGCN_REQUIRE(n_blocks >= 0 && (n_blocks == 0 || h_block4 != nullptr), "agcn_host_set_graph: null block4");
    AGCN_REQUIRE(nnz >= 0 && nnz <= (int64_t)INT32_MAX && (nnz == 0 || (h_indices != nullptr && h_vals != nullptr)),
                 "agcn_host_set_graph: null indices or values, or nnz out of range");
    AGCN_REQUIRE(n_rows > 0 && n_cols > 0, "agcn_host_set_graph: bad sizes");
    return AGCN_OK;
}

// Starts the upload of .block4 (the first thing the plan needs) on the upload stream.
static int upload_block4(agcn_host_ctx *c, const int *h_block4, int64_t n_blocks, int64_t n_rows, int64_t n_cols, int64_t nnz)
{
    plan_free(c->plan);
    c->plan = nullptr;
    c->n_rows = n_rows; c->n_cols = n_cols; c->nnz = nnz; c->n_blocks = n_blocks;
    const size_t bytes[3] = {(size_t)n_blocks * 16, (size_t)nnz * 4, (size_t)nnz * 4};
    for (int i = 0; i < 3; i++) {
        int rc = reserve(&c->graph[i], &c->graph_cap[i], bytes[i] > 0 ? bytes[i] : 16);
        if (rc != AGCN_OK) return rc;
    }
    if (c->d_abort == nullptr) AGCN_CUDA(cudaMalloc(&c->d_abort, sizeof(int)));
    AGCN_CUDA(cudaMemsetAsync(c->d_abort, 0, sizeof(int), c->s_run));
    if (n_blocks > 0) AGCN_CUDA(cudaMemcpyAsync(c->graph[0], h_block4, bytes[0], cudaMemcpyHostToDevice, c->s_up));
    return ctx_chain(c, c->s_up, c->s_run);
}

// Builds the plan from the uploaded .block4 (tuple validation, carry slots, uncovered rows;
// synchronises s_run) and fetches its carry bookkeeping for plan_parts.  Column ids are validated
// by the caller (whole array, or range by range as they arrive).
static int build_plan(agcn_host_ctx *c)
{
    int rc = spmm_create(&c->plan, static_cast<const int *>(c->graph[0]), c->n_blocks, nullptr, c->n_rows, c->n_cols, c->nnz, c->s_run);
    if (rc != AGCN_OK) return rc;
    c->h_unit_carry.assign((size_t)c->plan->n_units, make_int2(-1, -1));
    c->h_carry_row.assign((size_t)c->plan->n_carry, 0);
    if (c->plan->n_carry > 0) {
        AGCN_CUDA(cudaMemcpyAsync(c->h_unit_carry.data(), c->plan->unit_carry, c->h_unit_carry.size() * sizeof(int2),
                                  cudaMemcpyDeviceToHost, c->s_run));
        AGCN_CUDA(cudaMemcpyAsync(c->h_carry_row.data(), c->plan->carry_row, c->h_carry_row.size() * sizeof(int),
                                  cudaMemcpyDeviceToHost, c->s_run));
        AGCN_CUDA(cudaStreamSynchronize(c->s_run));
    }
    return AGCN_OK;
}

static int host_set_graph(agcn_host_ctx *c, const int *h_block4, int64_t n_blocks, const int *h_indices,
                          const float *h_vals, int64_t n_rows, int64_t n_cols, int64_t nnz)
{
    int rc = check_graph_args(c, h_block4, n_blocks, h_indices, h_vals, n_rows, n_cols, nnz);
    if (rc != AGCN_OK) return rc;
    // the column ids and values go up behind .block4 while the plan is being built from it
    rc = reserve(&c->graph[1], &c->graph_cap[1], nnz > 0 ? (size_t)nnz * 4 : 16);
    if (rc == AGCN_OK) rc = reserve(&c->graph[2], &c->graph_cap[2], nnz > 0 ? (size_t)nnz * 4 : 16);
    if (rc == AGCN_OK) rc = reserve(&c->graph[0], &c->graph_cap[0], n_blocks > 0 ? (size_t)n_blocks * 16 : 16);
    if (rc != AGCN_OK) return rc;
    rc = upload_block4(c, h_block4, n_blocks, n_rows, n_cols, nnz);
    if (rc != AGCN_OK) return rc;
    if (nnz > 0) AGCN_CUDA(cudaMemcpyAsync(c->graph[1], h_indices, (size_t)nnz * 4, cudaMemcpyHostToDevice, c->s_up));
    rc = build_plan(c);                   // on the host and s_run, while the column ids go up
    if (rc != AGCN_OK) { ctx_sync(c); return rc; }
    if (nnz > 0) {
        rc = ctx_chain(c, c->s_up, c->s_run);
        if (rc != AGCN_OK) return rc;
        rc = spmm_check_cols(static_cast<const int *>(c->graph[1]), nnz, n_cols, c->d_abort, c->s_run);   // under the upload of the values
        if (rc != AGCN_OK) return rc;
        AGCN_CUDA(cudaMemcpyAsync(c->graph[2], h_vals, (size_t)nnz * 4, cudaMemcpyHostToDevice, c->s_up));
    }
    int bad = 0;
    AGCN_CUDA(cudaMemcpyAsync(&bad, c->d_abort, sizeof(int), cudaMemcpyDeviceToHost, c->s_run));
    rc = ctx_sync(c);
    if (rc != AGCN_OK) return rc;
    if (bad != 0) {
        plan_free(c->plan);
        c->plan = nullptr;
        set_error("agcn_host_set_graph: invalid input: column index outside [0, n_cols);");
        return AGCN_ERR_RANGE;
    }
    plan_parts(c, h_block4, 4);
    return AGCN_OK;
}

static int reserve_products(agcn_host_ctx *c, int n, const int *dims, bool per_product_carry)
{
    if ((int)c->xbuf.size() < n) {
        c->xbuf.resize(n, nullptr); c->ybuf.resize(n, nullptr); c->cbuf.resize(n, nullptr);
        c->xcap.resize(n, 0); c->ycap.resize(n, 0); c->ccap.resize(n, 0);
    }
    for (int i = 0; i < n; i++) {
        int rc = reserve(&c->xbuf[i], &c->xcap[i], (size_t)c->n_cols * dims[i] * 4);
        if (rc == AGCN_OK) rc = reserve(&c->ybuf[i], &c->ycap[i], (size_t)c->n_rows * dims[i] * 4);
        // products whose unit ranges interleave each keep their own partial sums of the heavy rows
        if (rc == AGCN_OK && per_product_carry && c->plan->n_carry > 0)
            rc = reserve(&c->cbuf[i], &c->ccap[i], (size_t)c->plan->n_carry * HOST_SPMM_PANEL * 4);
        if (rc != AGCN_OK) return rc;
    }
    return AGCN_OK;
}

// rows [lo, hi) of product i: device -> host, on the download stream, after what s_run holds now
static int download_rows(agcn_host_ctx *c, int i, float *h_y, int dim, int64_t lo, int64_t hi)
{
    if (hi <= lo) return AGCN_OK;
    AGCN_CUDA(cudaMemcpyAsync(h_y + lo * dim, static_cast<const float *>(c->ybuf[i]) + lo * dim, (size_t)(hi - lo) * dim * 4,
                              cudaMemcpyDeviceToHost, c->s_down));
    return AGCN_OK;
}

static bool can_issue_in_parts(int dim) { return dim <= HOST_SPMM_PANEL && dim % 4 == 0; }

// Products on a graph that is already on the device: X_i up, product i in unit ranges, rows down as
// they complete.
static int host_products(agcn_host_ctx *c, int n, const float *const *h_x, float *const *h_y, const int *dims)
{
    AGCN_REQUIRE(c != nullptr && c->plan != nullptr, "agcn_host_spmm: no graph set (call agcn_host_set_graph first)");
    AGCN_REQUIRE(n >= 0 && (n == 0 || (h_x != nullptr && h_y != nullptr && dims != nullptr)), "agcn_host_spmm: null argument");
    for (int i = 0; i < n; i++)
        AGCN_REQUIRE(h_x[i] != nullptr && h_y[i] != nullptr && dims[i] >= 1, "agcn_host_spmm: null X or Y, or dim < 1");
    if (n == 0) return AGCN_OK;
    int rc = reserve_products(c, n, dims, false);
    if (rc != AGCN_OK) return rc;
    const int *idx = static_cast<const int *>(c->graph[1]);
    const float *val = static_cast<const float *>(c->graph[2]);
    std::vector<cudaEvent_t> x_up(n);
    for (int i = 0; i < n; i++) {
        AGCN_CUDA(cudaMemcpyAsync(c->xbuf[i], h_x[i], (size_t)c->n_cols * dims[i] * 4, cudaMemcpyHostToDevice, c->s_up));
        rc = ctx_event(c, &x_up[i]);
        if (rc != AGCN_OK) return rc;
        AGCN_CUDA(cudaEventRecord(x_up[i], c->s_up));
    }
    const int n_parts = (int)c->part_unit.size() - 1;
    for (int i = 0; i < n; i++) {
        const int dim = dims[i];
        float *y = static_cast<float *>(c->ybuf[i]);
        AGCN_CUDA(cudaStreamWaitEvent(c->s_run, x_up[i], 0));
        if (!can_issue_in_parts(dim) || n_parts <= 1) {
            rc = spmm_run(c->plan, idx, val, static_cast<const float *>(c->xbuf[i]), dim, y, dim, dim, c->s_run);
            if (rc == AGCN_OK) rc = ctx_chain(c, c->s_run, c->s_down);
            if (rc == AGCN_OK) rc = download_rows(c, i, h_y[i], dim, 0, c->n_rows);
            if (rc != AGCN_OK) { ctx_sync(c); return rc; }
            continue;
        }
        for (int k = 0; k < n_parts; k++) {
            // the units of the range, then the carry kernel over the rows the range completes
            SpmmLaunchPart part;
            part.unit0 = c->part_unit[k]; part.unit1 = c->part_unit[k + 1];
            part.zero_fill = k == 0;
            part.carry_s0 = c->part_slot[k]; part.carry_s1 = c->part_slot[k + 1];
            rc = spmm_run_prepared(c->plan, idx, val, static_cast<const float *>(c->xbuf[i]), dim, true, y, dim, dim, c->s_run, 0, 0, part);
            if (rc == AGCN_OK) rc = ctx_chain(c, c->s_run, c->s_down);
            if (rc == AGCN_OK) rc = download_rows(c, i, h_y[i], dim, c->part_row[k], c->part_row[k + 1]);
            if (rc != AGCN_OK) { ctx_sync(c); return rc; }
        }
    }
    return ctx_sync(c);
}

// The graph and the products in one call: A is uploaded in unit ranges and every range is
// multiplied for all products as soon as it is on the device.
static int host_graph_and_products(agcn_host_ctx *c, const int *h_block4, int64_t n_blocks, const int *h_indices,
                                   const float *h_vals, int64_t n_rows, int64_t n_cols, int64_t nnz, int n,
                                   const float *const *h_x, float *const *h_y, const int *dims)
{
    int rc = check_graph_args(c, h_block4, n_blocks, h_indices, h_vals, n_rows, n_cols, nnz);
    if (rc != AGCN_OK) return rc;
    AGCN_REQUIRE(n >= 0 && (n == 0 || (h_x != nullptr && h_y != nullptr && dims != nullptr)), "agcn_spmm_host_batch: null argument");
    bool stream_a = n > 0 && nnz > 0 && n_blocks > 0;
    for (int i = 0; i < n; i++) {
        AGCN_REQUIRE(h_x[i] != nullptr && h_y[i] != nullptr && dims[i] >= 1, "agcn_spmm_host_batch: null X or Y, or dim < 1");
        stream_a = stream_a && can_issue_in_parts(dims[i]);
    }
    if (!stream_a) {         // widths the unit-range launch does not take: graph first, then the products
        rc = host_set_graph(c, h_block4, n_blocks, h_indices, h_vals, n_rows, n_cols, nnz);
        return rc != AGCN_OK ? rc : host_products(c, n, h_x, h_y, dims);
    }
    const auto host_t0 = std::chrono::steady_clock::now();
    c->timed = false;
    AGCN_CUDA(cudaEventRecord(c->t_up0, c->s_up));
    // .block4 first, then every X behind it: the plan is built (on the host and on s_run) under those uploads
    rc = upload_block4(c, h_block4, n_blocks, n_rows, n_cols, nnz);
    if (rc == AGCN_OK) rc = reserve_products(c, n, dims, false);
    if (rc != AGCN_OK) { ctx_sync(c); return rc; }
    for (int i = 0; i < n; i++)
        AGCN_CUDA(cudaMemcpyAsync(c->xbuf[i], h_x[i], (size_t)n_cols * dims[i] * 4, cudaMemcpyHostToDevice, c->s_up));
    rc = build_plan(c);               // on the host and on s_run, under the uploads of X
    if (rc == AGCN_OK) rc = reserve_products(c, n, dims, true);       // now that the number of carry slots is known
    if (rc != AGCN_OK) { ctx_sync(c); return rc; }
    const auto host_t1 = std::chrono::steady_clock::now();
    // Column ids and values in ranges of about 32 MB: long enough for full PCIe speed, short enough
    // that the first product starts early and the last download is short.  Every upload is enqueued
    // before the first launch, so that the copy engine runs without a gap however long the host
    // takes over the launches below.  (Enqueued ahead of the plan build they delay it: its small
    // device-to-host copies then wait behind them.)
    plan_parts(c, h_block4, (int)std::max<int64_t>(1, std::min<int64_t>(64, (nnz * 8) >> 25)));
    const int n_parts = (int)c->part_unit.size() - 1;
    int *idx = static_cast<int *>(c->graph[1]);
    float *val = static_cast<float *>(c->graph[2]);
    std::vector<cudaEvent_t> part_up((size_t)n_parts);
    for (int k = 0; k < n_parts; k++) {
        const int64_t p0 = c->part_loc[k], p1 = c->part_loc[k + 1];
        AGCN_CUDA(cudaMemcpyAsync(idx + p0, h_indices + p0, (size_t)(p1 - p0) * 4, cudaMemcpyHostToDevice, c->s_up));
        AGCN_CUDA(cudaMemcpyAsync(val + p0, h_vals + p0, (size_t)(p1 - p0) * 4, cudaMemcpyHostToDevice, c->s_up));
        rc = ctx_event(c, &part_up[k]);
        if (rc != AGCN_OK) { ctx_sync(c); return rc; }
        AGCN_CUDA(cudaEventRecord(part_up[k], c->s_up));
    }
    AGCN_CUDA(cudaEventRecord(c->t_up1, c->s_up));
    for (int k = 0; k < n_parts; k++) {
        const int64_t p0 = c->part_loc[k], p1 = c->part_loc[k + 1];
        AGCN_CUDA(cudaStreamWaitEvent(c->s_run, part_up[k], 0));
        if (k == 0) AGCN_CUDA(cudaEventRecord(c->t_run0, c->s_run));
        // a column id outside [0, n_cols) sets the abort word, and every kernel behind it returns at once
        rc = spmm_check_cols(idx + p0, p1 - p0, n_cols, c->d_abort, c->s_run);
        for (int i = 0; i < n && rc == AGCN_OK; i++) {
            SpmmLaunchPart part;
            part.unit0 = c->part_unit[k]; part.unit1 = c->part_unit[k + 1];
            part.zero_fill = k == 0; part.abort_flag = c->d_abort;
            part.carry_s0 = c->part_slot[k]; part.carry_s1 = c->part_slot[k + 1];
            part.carry_buf = static_cast<float *>(c->cbuf[i]);
            rc = spmm_run_prepared(c->plan, idx, val, static_cast<const float *>(c->xbuf[i]), dims[i], true,
                                   static_cast<float *>(c->ybuf[i]), dims[i], dims[i], c->s_run, 0, 0, part);
        }
        if (rc == AGCN_OK) rc = ctx_chain(c, c->s_run, c->s_down);
        for (int i = 0; i < n && rc == AGCN_OK; i++)
            rc = download_rows(c, i, h_y[i], dims[i], c->part_row[k], c->part_row[k + 1]);
        if (rc != AGCN_OK) { ctx_sync(c); return rc; }
    }
    AGCN_CUDA(cudaEventRecord(c->t_run1, c->s_run));
    AGCN_CUDA(cudaEventRecord(c->t_down1, c->s_down));
    c->host_plan_ms = std::chrono::duration<float, std::milli>(host_t1 - host_t0).count();
    c->host_enqueue_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - host_t0).count();
    int bad = 0;
    if (rc == AGCN_OK && cudaMemcpyAsync(&bad, c->d_abort, sizeof(int), cudaMemcpyDeviceToHost, c->s_run) != cudaSuccess) rc = AGCN_ERR_CUDA;
    const int rc_sync = ctx_sync(c);
    if (rc != AGCN_OK || rc_sync != AGCN_OK) return rc != AGCN_OK ? rc : rc_sync;
    if (bad != 0) {
        plan_free(c->plan);
        c->plan = nullptr;
        set_error("agcn_spmm_host_batch: invalid input: column index outside [0, n_cols); the products were not computed");
        return AGCN_ERR_RANGE;
    }
    plan_parts(c, h_block4, 4);         // later agcn_host_spmm calls on this graph use a few large ranges
    c->timed = true;
    return AGCN_OK;
}

}  // namespace agcn

extern "C" int agcn_host_ctx_create(agcn_host_ctx **ctx)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(ctx != nullptr, "agcn_host_ctx_create: null pointer");
    *ctx = nullptr;
    agcn_host_ctx *c = new (std::nothrow) agcn_host_ctx;
    AGCN_REQUIRE(c != nullptr, "agcn_host_ctx_create: out of host memory");
    cudaError_t e = cudaStreamCreateWithFlags(&c->s_up, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->s_run, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->s_down, cudaStreamNonBlocking);
    for (cudaEvent_t *ev : {&c->t_up0, &c->t_up1, &c->t_run0, &c->t_run1, &c->t_down1})
        if (e == cudaSuccess) e = cudaEventCreate(ev);
    if (e != cudaSuccess) {
        agcn_host_ctx_destroy(c);
        set_error("agcn_host_ctx_create: cudaStreamCreate: %s", cudaGetErrorString(e));
        return AGCN_ERR_CUDA;
    }
    *ctx = c;
    return AGCN_OK;
}

extern "C" int agcn_host_ctx_destroy(agcn_host_ctx *ctx)
{
    agcn::clear_error();
    if (ctx == nullptr) return AGCN_OK;
    agcn::plan_free(ctx->plan);
    for (int i = 0; i < 3; i++) cudaFree(ctx->graph[i]);
    for (void *p : ctx->xbuf) cudaFree(p);
    for (void *p : ctx->ybuf) cudaFree(p);
    for (void *p : ctx->cbuf) cudaFree(p);
    cudaFree(ctx->d_abort);
    for (cudaEvent_t e : ctx->events) cudaEventDestroy(e);
    for (cudaEvent_t e : {ctx->t_up0, ctx->t_up1, ctx->t_run0, ctx->t_run1, ctx->t_down1}) if (e) cudaEventDestroy(e);
    if (ctx->s_up) cudaStreamDestroy(ctx->s_up);
    if (ctx->s_run) cudaStreamDestroy(ctx->s_run);
    if (ctx->s_down) cudaStreamDestroy(ctx->s_down);
    delete ctx;
    return AGCN_OK;
}

extern "C" int agcn_host_set_graph(agcn_host_ctx *ctx, const int32_t *h_block4, int64_t n_blocks,
                                   const int32_t *h_indices, const float *h_vals,
                                   int64_t n_rows, int64_t n_cols, int64_t nnz)
{
    agcn::clear_error();
    return agcn::host_set_graph(ctx, h_block4, n_blocks, h_indices, h_vals, n_rows, n_cols, nnz);
}

extern "C" int agcn_host_spmm(agcn_host_ctx *ctx, const float *h_x, float *h_y, int dim)
{
    agcn::clear_error();
    return agcn::host_products(ctx, 1, &h_x, &h_y, &dim);
}

extern "C" int agcn_host_spmm_batch(agcn_host_ctx *ctx, int n_products, const float *const *h_x, float *const *h_y,
                                    const int *dims)
{
    agcn::clear_error();
    return agcn::host_products(ctx, n_products, h_x, h_y, dims);
}

extern "C" int agcn_spmm_host(agcn_host_ctx *ctx, const int32_t *h_block4, int64_t n_blocks,
                              const int32_t *h_indices, const float *h_vals, const float *h_x, float *h_y,
                              int64_t n_rows, int64_t n_cols, int64_t nnz, int dim)
{
    agcn::clear_error();
    return agcn::host_graph_and_products(ctx, h_block4, n_blocks, h_indices, h_vals, n_rows, n_cols, nnz, 1, &h_x, &h_y, &dim);
}

extern "C" int agcn_spmm_host_batch(agcn_host_ctx *ctx, const int32_t *h_block4, int64_t n_blocks,
                                    const int32_t *h_indices, const float *h_vals,
                                    int64_t n_rows, int64_t n_cols, int64_t nnz,
                                    int n_products, const float *const *h_x, float *const *h_y, const int *dims)
{
    agcn::clear_error();
    return agcn::host_graph_and_products(ctx, h_block4, n_blocks, h_indices, h_vals, n_rows, n_cols, nnz, n_products, h_x, h_y, dims);
}

// Where the time of the last agcn_spmm_host_batch call on this context went, in milliseconds from
// the start of its uploads: [0] last byte of A uploaded, [1] first kernel started, [2] last kernel
// finished, [3] last byte of Y downloaded; then host-side times: [4] until the plan was built,
// [5] until everything was enqueued.
extern "C" int agcn_host_last_timing(agcn_host_ctx *ctx, float *ms6)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(ctx != nullptr && ms6 != nullptr, "agcn_host_last_timing: null argument");
    AGCN_REQUIRE(ctx->timed, "agcn_host_last_timing: no streamed agcn_spmm_host_batch call has completed on this context");
    AGCN_CUDA(cudaEventElapsedTime(&ms6[0], ctx->t_up0, ctx->t_up1));
    AGCN_CUDA(cudaEventElapsedTime(&ms6[1], ctx->t_up0, ctx->t_run0));
    AGCN_CUDA(cudaEventElapsedTime(&ms6[2], ctx->t_up0, ctx->t_run1));
    AGCN_CUDA(cudaEventElapsedTime(&ms6[3], ctx->t_up0, ctx->t_down1));
    ms6[4] = ctx->host_plan_ms;
    ms6[5] = ctx->host_enqueue_ms;
    return AGCN_OK;
}
