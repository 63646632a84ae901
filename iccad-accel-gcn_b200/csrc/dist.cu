// Row-sharded multi-GPU SpMM and the two-layer GCN forward behind the C ABI
// (agcn_dist_*, agcn_gcn2_forward_*): one process (or thread) per GPU, NCCL for the one exchange
// the path has -- the all-gather of the dense operand.  The reference is single-GPU
// (main.cu:53-182); this is its operator, spmm_accel.cu, applied block by block.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy the process already has loaded if
// any), so the library carries no link-time dependency and single-GPU users never load it.
#include "host_common.h"
#include "internal.h"
#include "kernels/dist_kernels.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <new>
#include <vector>

typedef struct agcn_spmm_tiled agcn_spmm_tiled;
extern "C" int agcn_spmm_tiled_create(agcn_spmm_tiled **plan, const int32_t *d_indptr, const int32_t *d_indices,
                                      const float *d_vals, int64_t n_rows, int64_t n_cols, int64_t nnz,
                                      const int32_t *h_bounds, int n_ranges, void *stream);
extern "C" int agcn_spmm_tiled_run_range(agcn_spmm_tiled *plan, int range, const float *d_x, int64_t ldx, float *d_y,
                                         int64_t ldy, int dim, int activation, void *stream);
extern "C" int agcn_spmm_tiled_destroy(agcn_spmm_tiled *plan);
extern "C" int agcn_spmm_tiled_info(const agcn_spmm_tiled *plan, int *n_ranges, int64_t *n_blocks_total, int64_t *range_nnz,
                                    int *launches_last_run);

namespace agcn {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

static int nccl_api(const NcclApi **out)
{
    static std::mutex mutex;
    static NcclApi api;
    std::lock_guard<std::mutex> lock(mutex);
    if (api.handle == nullptr) {
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) {
            set_error("agcn_dist: cannot load libnccl.so.2 (%s)", dlerror());
            return AGCN_ERR_CUDA;
        }
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllGather || !api.GetErrorString) {
            set_error("agcn_dist: libnccl.so.2 lacks a needed symbol");
            dlclose(h);
            return AGCN_ERR_CUDA;
        }
        api.handle = h;
    }
    *out = &api;
    return AGCN_OK;
}

#define AGCN_NCCL(api, call)                                                                        \
    do {                                                                                            \
        ncclResult_t agcn_r_ = (call);                                                              \
        if (agcn_r_ != ncclSuccess) {                                                               \
            ::agcn::set_error("%s: %s (%s:%d)", #call, (api)->GetErrorString(agcn_r_), __FILE__, __LINE__); \
            return AGCN_ERR_CUDA;                                                                   \
        }                                                                                           \
    } while (0)

constexpr int DIST_SLOTS = 4;             // gathered operands that can be in flight at once
constexpr int DIST_MAX_CHUNKS = 16;

}  // namespace agcn

struct agcn_dist {
    int rank = 0, world = 1, chunks = 1, ranges = 1;     // exchange slices; column ranges of the block's tiled plan
    const agcn::NcclApi *nccl = nullptr;
    ncclComm_t comm = nullptr;
    cudaStream_t s_comm = nullptr;
    // this rank's block of A
    agcn::DistLayout layout;
    int64_t n = 0, per = 0, n_gathered = 0, local_rows = 0, local_nnz = 0, n_blocks = 0;
    int *indptr = nullptr, *idx = nullptr, *block4 = nullptr;
    float *val = nullptr;
    agcn_spmm_plan *plan = nullptr;           // ranges == 1
    agcn_spmm_tiled *tiled = nullptr;         // ranges > 1: one column range per exchanged slice, or equal ranges of the gathered operand
    // gathered operands
    float *gathered[agcn::DIST_SLOTS] = {};
    size_t gathered_cap[agcn::DIST_SLOTS] = {};
    const float *gathered_ptr[agcn::DIST_SLOTS] = {};     // what the SpMM reads (the caller's block itself when world == 1)
    int gathered_dim[agcn::DIST_SLOTS] = {};
    cudaEvent_t ev_ready[agcn::DIST_SLOTS][agcn::DIST_MAX_CHUNKS] = {};     // slice c of slot s has arrived
    cudaEvent_t ev_consumed[agcn::DIST_SLOTS] = {};                        // the last SpMM reading slot s has finished
    cudaEvent_t ev_input = nullptr;                                        // the caller's block is ready on its stream
    bool slot_used[agcn::DIST_SLOTS] = {};
    int launches_last_step = 0;
};

struct agcn_gcn2 {
    agcn_dist *dist = nullptr;
    const float *w[2] = {nullptr, nullptr};
    float *z = nullptr, *h1 = nullptr;        // [per x 128] each
    int *d_status = nullptr;                  // status words: the GEMM of each layer, the fused kernel, the GEMM of the other rows
    cudaEvent_t ev[8] = {};
    // AGCN_GCN_FUSED=1: the leading rows of the block (at most 32 nonzeros each) go through one kernel
    // from layer 1's gathered operand to layer 2's operand; the other rows through SpMM and GEMM as before
    float *z2 = nullptr;                      // [per x 128]: layer 2's operand
    int64_t fused_rows = 0;                   // rows [0, fused_rows) are the fused kernel's
    int64_t rest_unit = 0;                    // first unit of the SpMM over the other rows (it may start a few rows early)
};

namespace agcn {

static void dist_free_graph(agcn_dist *d)
{
    plan_free(d->plan); d->plan = nullptr;
    if (d->tiled != nullptr) agcn_spmm_tiled_destroy(d->tiled);
    d->tiled = nullptr;
    cudaFree(d->indptr); cudaFree(d->idx); cudaFree(d->val); cudaFree(d->block4);
    d->indptr = d->idx = d->block4 = nullptr; d->val = nullptr;
}

static void dist_free(agcn_dist *d)
{
    if (d == nullptr) return;
    dist_free_graph(d);
    for (int s = 0; s < DIST_SLOTS; s++) {
        cudaFree(d->gathered[s]);
        for (int c = 0; c < DIST_MAX_CHUNKS; c++) if (d->ev_ready[s][c]) cudaEventDestroy(d->ev_ready[s][c]);
        if (d->ev_consumed[s]) cudaEventDestroy(d->ev_consumed[s]);
    }
    if (d->ev_input) cudaEventDestroy(d->ev_input);
    if (d->comm != nullptr && d->nccl != nullptr) d->nccl->CommDestroy(d->comm);
    if (d->s_comm) cudaStreamDestroy(d->s_comm);
    delete d;
}

static int dist_create(agcn_dist **out, int rank, int world, const void *id)
{
    AGCN_REQUIRE(out != nullptr, "agcn_dist_create: null pointer");
    *out = nullptr;
    AGCN_REQUIRE(world >= 1 && world <= DIST_MAX_WORLD && rank >= 0 && rank < world, "agcn_dist_create: rank %d of %d", rank, world);
    agcn_dist *d = new (std::nothrow) agcn_dist;
    AGCN_REQUIRE(d != nullptr, "agcn_dist_create: out of host memory");
    struct Guard { agcn_dist *d; ~Guard() { dist_free(d); } } guard{d};
    d->rank = rank; d->world = world;
    AGCN_CUDA(cudaStreamCreateWithFlags(&d->s_comm, cudaStreamNonBlocking));
    AGCN_CUDA(cudaEventCreateWithFlags(&d->ev_input, cudaEventDisableTiming));
    for (int s = 0; s < DIST_SLOTS; s++) {
        for (int c = 0; c < DIST_MAX_CHUNKS; c++) AGCN_CUDA(cudaEventCreateWithFlags(&d->ev_ready[s][c], cudaEventDisableTiming));
        AGCN_CUDA(cudaEventCreateWithFlags(&d->ev_consumed[s], cudaEventDisableTiming));
    }
    if (world > 1 && id != nullptr) {
        int rc = nccl_api(&d->nccl);
        if (rc != AGCN_OK) return rc;
        ncclUniqueId uid;
        static_assert(sizeof(uid) == AGCN_DIST_ID_BYTES, "AGCN_DIST_ID_BYTES must be sizeof(ncclUniqueId)");
        memcpy(&uid, id, sizeof(uid));
        AGCN_NCCL(d->nccl, d->nccl->CommInitRank(&d->comm, world, uid, rank));
    }
    guard.d = nullptr;
    *out = d;
    return AGCN_OK;
}

// Builds this rank's block from the whole degree-ordered matrix on this device.
static int dist_set_graph(agcn_dist *d, const int *d_indptr, const int *d_indices, const float *d_vals, int64_t n_rows,
                          int64_t nnz, int chunks, int column_ranges, cudaStream_t s)
{
    AGCN_REQUIRE(d != nullptr, "agcn_dist_set_graph: null context");
    AGCN_REQUIRE(d_indptr != nullptr && n_rows > 0 && n_rows < (int64_t)INT32_MAX / 2, "agcn_dist_set_graph: null indptr or bad n_rows");
    AGCN_REQUIRE(nnz >= 0 && nnz <= (int64_t)INT32_MAX && (nnz == 0 || (d_indices != nullptr && d_vals != nullptr)),
                 "agcn_dist_set_graph: bad nnz, or null indices / values");
    AGCN_REQUIRE(chunks >= 1 && chunks <= DIST_MAX_CHUNKS && chunks <= 32, "agcn_dist_set_graph: 1..%d exchange slices", DIST_MAX_CHUNKS);
    AGCN_REQUIRE(column_ranges >= 1 && column_ranges <= 32, "agcn_dist_set_graph: 1..32 column ranges");
    dist_free_graph(d);
    for (int sl = 0; sl < DIST_SLOTS; sl++) d->slot_used[sl] = false;

    // layout from a host copy of the row pointers (the same on every rank)
    std::vector<int> h_indptr((size_t)n_rows + 1);
    AGCN_CUDA(cudaMemcpyAsync(h_indptr.data(), d_indptr, ((size_t)n_rows + 1) * sizeof(int), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaStreamSynchronize(s));
    AGCN_REQUIRE(h_indptr[0] == 0 && (int64_t)h_indptr[n_rows] == nnz, "agcn_dist_set_graph: indptr must run from 0 to nnz");
    std::vector<int64_t> ranges((size_t)d->world * 4);
    int64_t per = 0;
    int rc = balanced_blocks(h_indptr.data(), n_rows, d->world, ranges.data(), &per);
    if (rc != AGCN_OK) return rc;
    if (d->world == 1) chunks = 1;                      // nothing is exchanged
    per = ceil_div(per, chunks) * chunks;               // slices of equal height
    DistLayout &L = d->layout;
    L.world = d->world; L.chunks = chunks; L.per = (int)per; L.rows_per_chunk = (int)(per / chunks);
    for (int g = 0; g < d->world; g++) {
        L.light0[g] = (int)ranges[4 * g + 0]; L.light1[g] = (int)ranges[4 * g + 1];
        L.heavy0[g] = (int)ranges[4 * g + 2]; L.heavy1[g] = (int)ranges[4 * g + 3];
    }
    const int g = d->rank;
    d->chunks = chunks; d->n = n_rows; d->per = per; d->n_gathered = per * d->world;
    d->local_rows = (L.light1[g] - L.light0[g]) + (L.heavy1[g] - L.heavy0[g]);
    const int64_t light_nz = (int64_t)h_indptr[L.light1[g]] - h_indptr[L.light0[g]];
    const int64_t heavy_nz = (int64_t)h_indptr[L.heavy1[g]] - h_indptr[L.heavy0[g]];
    d->local_nnz = light_nz + heavy_nz;

    AGCN_CUDA(cudaMalloc(&d->indptr, ((size_t)per + 1) * sizeof(int)));
    AGCN_CUDA(cudaMalloc(&d->idx, (size_t)(d->local_nnz > 0 ? d->local_nnz : 1) * sizeof(int)));
    AGCN_CUDA(cudaMalloc(&d->val, (size_t)(d->local_nnz > 0 ? d->local_nnz : 1) * sizeof(float)));
    AGCN_KERNEL(dist_local_indptr_kernel, (unsigned)ceil_div(per + 1, 256), 256, s, d_indptr, L, g, d->indptr);
    AGCN_LAUNCH_CHECK("dist_local_indptr_kernel");
    if (light_nz > 0) {
        AGCN_CUDA(cudaMemcpyAsync(d->idx, d_indices + h_indptr[L.light0[g]], (size_t)light_nz * 4, cudaMemcpyDeviceToDevice, s));
        AGCN_CUDA(cudaMemcpyAsync(d->val, d_vals + h_indptr[L.light0[g]], (size_t)light_nz * 4, cudaMemcpyDeviceToDevice, s));
    }
    if (heavy_nz > 0) {
        AGCN_CUDA(cudaMemcpyAsync(d->idx + light_nz, d_indices + h_indptr[L.heavy0[g]], (size_t)heavy_nz * 4, cudaMemcpyDeviceToDevice, s));
        AGCN_CUDA(cudaMemcpyAsync(d->val + light_nz, d_vals + h_indptr[L.heavy0[g]], (size_t)heavy_nz * 4, cudaMemcpyDeviceToDevice, s));
    }
    // column ids -> positions in the gathered operand
    DeviceScratch scratch;
    AGCN_ALLOC(d_err, scratch, int, 1);
    AGCN_CUDA(cudaMemsetAsync(d_err, 0, sizeof(int), s));
    if (d->local_nnz > 0) {
        const int64_t blocks = ceil_div(d->local_nnz, 256 * 8);
        AGCN_KERNEL(dist_relabel_kernel, (unsigned)(blocks < 65535 ? blocks : 65535), 256, s, d->idx, d->local_nnz, (int)n_rows, L, d_err);
        AGCN_LAUNCH_CHECK("dist_relabel_kernel");
    }
    int err = 0;
    AGCN_CUDA(cudaMemcpyAsync(&err, d_err, sizeof(int), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaStreamSynchronize(s));
    if (err != 0) {
        set_error("agcn_dist_set_graph: a column id lies outside [0, n_rows): the matrix must be square");
        return AGCN_ERR_RANGE;
    }

    // sliced exchange: one column range per slice; otherwise the caller's choice of equal ranges
    d->ranges = chunks > 1 ? chunks : column_ranges;
    if (d->ranges == 1) {
        rc = partition_device(d->indptr, per, nullptr, 0, &d->n_blocks, s);
        if (rc != AGCN_OK) return rc;
        if (d->n_blocks > 0) {
            AGCN_CUDA(cudaMalloc(&d->block4, (size_t)d->n_blocks * 16));
            rc = partition_device(d->indptr, per, d->block4, d->n_blocks, &d->n_blocks, s);
            if (rc != AGCN_OK) return rc;
        }
        return spmm_create(&d->plan, d->block4, d->n_blocks, d->idx, per, d->n_gathered, d->local_nnz, s);
    }
    // with a sliced exchange the product over a slice starts when that slice has arrived; with column
    // ranges alone every launch gathers from one L2-sized slab of the gathered operand
    std::vector<int> bounds((size_t)d->ranges + 1);
    for (int c = 0; c <= d->ranges; c++)
        bounds[c] = chunks > 1 ? (int)((int64_t)c * d->world * L.rows_per_chunk) : (int)(d->n_gathered * c / d->ranges);
    rc = agcn_spmm_tiled_create(&d->tiled, d->indptr, d->idx, d->val, per, d->n_gathered, d->local_nnz, bounds.data(), d->ranges, s);
    if (rc != AGCN_OK) return rc;
    return agcn_spmm_tiled_info(d->tiled, nullptr, &d->n_blocks, nullptr, nullptr);
}

static int dist_gather_begin(agcn_dist *d, int slot, const float *d_x_block, int dim, cudaStream_t s)
{
    AGCN_REQUIRE(d != nullptr && (d->plan != nullptr || d->tiled != nullptr), "agcn_dist_gather_begin: no graph set");
    AGCN_REQUIRE(slot >= 0 && slot < DIST_SLOTS, "agcn_dist_gather_begin: slot %d outside 0..%d", slot, DIST_SLOTS - 1);
    AGCN_REQUIRE(d_x_block != nullptr && dim >= 1, "agcn_dist_gather_begin: null block or dim < 1");
    d->gathered_dim[slot] = dim;
    if (d->world == 1) {
        d->gathered_ptr[slot] = d_x_block;        // the block is the whole operand
        d->slot_used[slot] = true;
        AGCN_CUDA(cudaEventRecord(d->ev_ready[slot][0], s));
        return AGCN_OK;
    }
    AGCN_REQUIRE(d->comm != nullptr, "agcn_dist_gather_begin: the context was created without a communicator (id = NULL): "
                                     "exchange the operand yourself and call agcn_dist_spmm_on_gathered");
    const size_t need = (size_t)d->n_gathered * dim * sizeof(float);
    if (need > d->gathered_cap[slot]) {
        if (d->gathered[slot] != nullptr) AGCN_CUDA(cudaFree(d->gathered[slot]));
        d->gathered[slot] = nullptr; d->gathered_cap[slot] = 0;
        AGCN_CUDA(cudaMalloc(&d->gathered[slot], need));
        d->gathered_cap[slot] = need;
        d->slot_used[slot] = false;
    }
    d->gathered_ptr[slot] = d->gathered[slot];
    // the exchange starts when the caller's block is ready and the buffer's last reader is done
    AGCN_CUDA(cudaEventRecord(d->ev_input, s));
    AGCN_CUDA(cudaStreamWaitEvent(d->s_comm, d->ev_input, 0));
    if (d->slot_used[slot]) AGCN_CUDA(cudaStreamWaitEvent(d->s_comm, d->ev_consumed[slot], 0));
    const int64_t slice_rows = d->layout.rows_per_chunk;
    for (int c = 0; c < d->chunks; c++) {
        const float *src = d_x_block + (int64_t)c * slice_rows * dim;
        float *dst = d->gathered[slot] + (int64_t)c * d->world * slice_rows * dim;
        AGCN_NCCL(d->nccl, d->nccl->AllGather(src, dst, (size_t)slice_rows * dim, ncclFloat, d->comm, d->s_comm));
        AGCN_CUDA(cudaEventRecord(d->ev_ready[slot][c], d->s_comm));
    }
    d->slot_used[slot] = true;
    return AGCN_OK;
}

static int dist_spmm_gathered(agcn_dist *d, int slot, float *d_y_block, int dim, int activation, cudaStream_t s)
{
    AGCN_REQUIRE(d != nullptr && (d->plan != nullptr || d->tiled != nullptr), "agcn_dist_spmm_gathered: no graph set");
    AGCN_REQUIRE(slot >= 0 && slot < DIST_SLOTS && d->slot_used[slot] && d->gathered_dim[slot] == dim,
                 "agcn_dist_spmm_gathered: slot %d holds no gathered operand of %d columns", slot, dim);
    AGCN_REQUIRE(d_y_block != nullptr, "agcn_dist_spmm_gathered: null output");
    const float *x = d->gathered_ptr[slot];
    d->launches_last_step = 0;
    int rc = AGCN_OK;
    if (d->tiled == nullptr) {
        AGCN_CUDA(cudaStreamWaitEvent(s, d->ev_ready[slot][0], 0));
        rc = spmm_run(d->plan, d->idx, d->val, x, dim, d_y_block, dim, dim, s, activation, 0);
        d->launches_last_step = d->plan->launches_last_run;
    } else {
        for (int c = 0; c < d->ranges && rc == AGCN_OK; c++) {
            if (c < d->chunks) AGCN_CUDA(cudaStreamWaitEvent(s, d->ev_ready[slot][c], 0));
            rc = agcn_spmm_tiled_run_range(d->tiled, c, x, dim, d_y_block, dim, dim, activation, s);
        }
        int launches = 0;
        if (rc == AGCN_OK) rc = agcn_spmm_tiled_info(d->tiled, nullptr, nullptr, nullptr, &launches);
        d->launches_last_step = launches;
    }
    if (rc != AGCN_OK) return rc;
    AGCN_CUDA(cudaEventRecord(d->ev_consumed[slot], s));
    return AGCN_OK;
}

// The local product on an operand the caller has assembled itself ([world * rows_per_block x dim]
// in gathered order): for callers with their own exchange, and for running every rank's block in
// one process.
static int dist_spmm_on_gathered(agcn_dist *d, const float *d_gathered, float *d_y_block, int dim, int activation, cudaStream_t s)
{
    AGCN_REQUIRE(d != nullptr && (d->plan != nullptr || d->tiled != nullptr), "agcn_dist_spmm_on_gathered: no graph set");
    AGCN_REQUIRE(d_gathered != nullptr && d_y_block != nullptr && dim >= 1, "agcn_dist_spmm_on_gathered: null operand or dim < 1");
    int rc = AGCN_OK;
    if (d->tiled == nullptr) {
        rc = spmm_run(d->plan, d->idx, d->val, d_gathered, dim, d_y_block, dim, dim, s, activation, 0);
        d->launches_last_step = d->plan->launches_last_run;
    } else {
        for (int c = 0; c < d->ranges && rc == AGCN_OK; c++)
            rc = agcn_spmm_tiled_run_range(d->tiled, c, d_gathered, dim, d_y_block, dim, dim, activation, s);
        int launches = 0;
        if (rc == AGCN_OK) rc = agcn_spmm_tiled_info(d->tiled, nullptr, nullptr, nullptr, &launches);
        d->launches_last_step = launches;
    }
    return rc;
}

static void gcn2_free(agcn_gcn2 *f)
{
    if (f == nullptr) return;
    cudaFree(f->z); cudaFree(f->h1); cudaFree(f->z2); cudaFree(f->d_status);
    for (cudaEvent_t e : f->ev) if (e) cudaEventDestroy(e);
    delete f;
}

}  // namespace agcn

extern "C" int agcn_dist_unique_id(void *id)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(id != nullptr, "agcn_dist_unique_id: null pointer");
    const NcclApi *api = nullptr;
    int rc = nccl_api(&api);
    if (rc != AGCN_OK) return rc;
    ncclUniqueId uid;
    AGCN_NCCL(api, api->GetUniqueId(&uid));
    memcpy(id, &uid, sizeof(uid));
    return AGCN_OK;
}

extern "C" int agcn_dist_create(agcn_dist **dist, int rank, int world, const void *id)
{
    agcn::clear_error();
    return agcn::dist_create(dist, rank, world, id);
}

extern "C" int agcn_dist_destroy(agcn_dist *dist)
{
    agcn::clear_error();
    agcn::dist_free(dist);
    return AGCN_OK;
}

extern "C" int agcn_dist_set_graph(agcn_dist *dist, const int32_t *d_indptr, const int32_t *d_indices, const float *d_vals,
                                   int64_t n_rows, int64_t nnz, int exchange_slices, int column_ranges, void *stream)
{
    agcn::clear_error();
    int rc = agcn::dist_set_graph(dist, d_indptr, d_indices, d_vals, n_rows, nnz, exchange_slices, column_ranges,
                                  static_cast<cudaStream_t>(stream));
    if (rc != AGCN_OK && dist != nullptr) agcn::dist_free_graph(dist);
    return rc;
}

extern "C" int agcn_dist_info(const agcn_dist *dist, int64_t *rows_per_block, int64_t *local_rows, int64_t *local_nnz,
                              int64_t *n_blocks, int *exchange_slices, int *launches_last_step)
{
    agcn::clear_error();
    AGCN_REQUIRE(dist != nullptr, "agcn_dist_info: null context");
    if (rows_per_block) *rows_per_block = dist->per;
    if (local_rows) *local_rows = dist->local_rows;
    if (local_nnz) *local_nnz = dist->local_nnz;
    if (n_blocks) *n_blocks = dist->n_blocks;
    if (exchange_slices) *exchange_slices = dist->chunks;
    if (launches_last_step) *launches_last_step = dist->launches_last_step;
    return AGCN_OK;
}

extern "C" int agcn_dist_block_rows(const agcn_dist *dist, int rank, int32_t *d_rows, void *stream)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(dist != nullptr && dist->per > 0 && d_rows != nullptr, "agcn_dist_block_rows: no graph set, or null output");
    AGCN_REQUIRE(rank >= 0 && rank < dist->world, "agcn_dist_block_rows: rank %d of %d", rank, dist->world);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    AGCN_KERNEL(dist_block_rows_kernel, (unsigned)ceil_div(dist->per, 256), 256, s, dist->layout, rank, d_rows);
    AGCN_LAUNCH_CHECK("dist_block_rows_kernel");
    return AGCN_OK;
}

extern "C" int agcn_dist_gather_begin(agcn_dist *dist, int slot, const float *d_x_block, int dim, void *stream)
{
    agcn::clear_error();
    return agcn::dist_gather_begin(dist, slot, d_x_block, dim, static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_dist_spmm_gathered(agcn_dist *dist, int slot, float *d_y_block, int dim, int activation, void *stream)
{
    agcn::clear_error();
    return agcn::dist_spmm_gathered(dist, slot, d_y_block, dim, activation, static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_dist_wait_gathered(agcn_dist *dist, int slot, void *stream)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(dist != nullptr && slot >= 0 && slot < DIST_SLOTS && dist->slot_used[slot], "agcn_dist_wait_gathered: empty slot");
    const int n = dist->world == 1 ? 1 : dist->chunks;
    for (int c = 0; c < n; c++) AGCN_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), dist->ev_ready[slot][c], 0));
    return AGCN_OK;
}

extern "C" int agcn_dist_spmm_step(agcn_dist *dist, const float *d_x_block, float *d_y_block, int dim, int activation,
                                   void *stream)
{
    agcn::clear_error();
    int rc = agcn::dist_gather_begin(dist, 0, d_x_block, dim, static_cast<cudaStream_t>(stream));
    if (rc != AGCN_OK) return rc;
    return agcn::dist_spmm_gathered(dist, 0, d_y_block, dim, activation, static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_dist_spmm_on_gathered(agcn_dist *dist, const float *d_gathered, float *d_y_block, int dim,
                                          int activation, void *stream)
{
    agcn::clear_error();
    return agcn::dist_spmm_on_gathered(dist, d_gathered, d_y_block, dim, activation, static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_dist_gathered(const agcn_dist *dist, int slot, const float **d_gathered, int64_t *n_rows)
{
    agcn::clear_error();
    AGCN_REQUIRE(dist != nullptr && slot >= 0 && slot < agcn::DIST_SLOTS && dist->slot_used[slot], "agcn_dist_gathered: empty slot");
    if (d_gathered) *d_gathered = dist->gathered_ptr[slot];
    if (n_rows) *n_rows = dist->world == 1 ? dist->per : dist->n_gathered;
    return AGCN_OK;
}

// ---------------------------------------------------------------------------
// two-layer GCN forward  relu(A relu(A X W1) W2)  on the row blocks
// ---------------------------------------------------------------------------
extern "C" int agcn_gcn2_forward_create(agcn_gcn2 **fwd, agcn_dist *dist, const float *d_w1, const float *d_w2)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(fwd != nullptr, "agcn_gcn2_forward_create: null pointer");
    *fwd = nullptr;
    AGCN_REQUIRE(dist != nullptr && (dist->plan != nullptr || dist->tiled != nullptr), "agcn_gcn2_forward_create: the context has no graph");
    AGCN_REQUIRE(d_w1 != nullptr && d_w2 != nullptr, "agcn_gcn2_forward_create: null weights");
    agcn_gcn2 *f = new (std::nothrow) agcn_gcn2;
    AGCN_REQUIRE(f != nullptr, "agcn_gcn2_forward_create: out of host memory");
    struct Guard { agcn_gcn2 *f; ~Guard() { gcn2_free(f); } } guard{f};
    f->dist = dist; f->w[0] = d_w1; f->w[1] = d_w2;
    const size_t bytes = (size_t)dist->per * 128 * sizeof(float);
    AGCN_CUDA(cudaMalloc(&f->z, bytes));
    AGCN_CUDA(cudaMalloc(&f->h1, bytes));
    AGCN_CUDA(cudaMalloc(&f->d_status, 4 * sizeof(int)));
    AGCN_CUDA(cudaMemset(f->d_status, 0, 4 * sizeof(int)));
    for (cudaEvent_t &e : f->ev) AGCN_CUDA(cudaEventCreate(&e));
    if (env_int("AGCN_GCN_FUSED", 0) != 0 && dist->plan != nullptr && dist->per > 0 && dist->n_blocks > 0) {
        // leading rows of at most 32 nonzeros (the block starts with its light rows in ascending degree), in whole tiles
        std::vector<int> h_indptr((size_t)dist->per + 1);
        AGCN_CUDA(cudaMemcpy(h_indptr.data(), dist->indptr, h_indptr.size() * sizeof(int), cudaMemcpyDeviceToHost));
        int64_t rows = 0;
        while (rows < dist->per && h_indptr[rows + 1] - h_indptr[rows] <= fused_layer_max_degree()) rows++;
        rows -= rows % 128;
        // the unit (8 tuples) that holds the first row left to the SpMM: first rows of every unit's first tuple
        const int64_t n_units = ceil_div(dist->n_blocks, 8);
        std::vector<int> unit_row((size_t)n_units);
        AGCN_CUDA(cudaMemcpy2D(unit_row.data(), sizeof(int), dist->block4 + 1, 8 * 4 * sizeof(int), sizeof(int), (size_t)n_units,
                               cudaMemcpyDeviceToHost));
        int64_t lo = 0, hi = n_units;                    // first unit whose first row is > rows
        while (lo < hi) {
            const int64_t mid = lo + (hi - lo) / 2;
            if (unit_row[mid] <= rows) lo = mid + 1; else hi = mid;
        }
        if (rows >= 128 * 64 && lo > 0) {
            f->fused_rows = rows;
            f->rest_unit = lo - 1;
            AGCN_CUDA(cudaMalloc(&f->z2, bytes));
        }
    }
    guard.f = nullptr;
    *fwd = f;
    return AGCN_OK;
}

// Enqueues one forward on `stream` and returns without waiting.  d_x_block / d_out_block are this
// rank's rows [rows_per_block x 128] (padding rows zero).  Per layer: Z = H * W on the tensor
// cores, all-gather of Z on the communication stream (slice by slice), relu(A_block * Z).
extern "C" int agcn_gcn2_forward_run(agcn_gcn2 *fwd, const float *d_x_block, float *d_out_block, void *stream)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(fwd != nullptr && d_x_block != nullptr && d_out_block != nullptr, "agcn_gcn2_forward_run: null argument");
    agcn_dist *d = fwd->dist;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float *h = d_x_block;
    const bool fused = fwd->fused_rows > 0;
    for (int layer = 0; layer < 2; layer++) {
        float *out = layer == 0 ? fwd->h1 : d_out_block;
        const float *operand = fwd->z;
        AGCN_CUDA(cudaEventRecord(fwd->ev[4 * layer + 0], s));
        int rc = AGCN_OK;
        if (fused && layer == 1) operand = fwd->z2;        // made by layer 1's fused step
        else rc = gemm_tf32_async(h, 128, fwd->w[layer], fwd->z, 128, d->per, fwd->d_status + layer, s);
        if (rc != AGCN_OK) return rc;
        AGCN_CUDA(cudaEventRecord(fwd->ev[4 * layer + 1], s));
        rc = dist_gather_begin(d, 0, operand, 128, s);
        if (rc == AGCN_OK && fused && layer == 0) {
            // light rows: relu(A Z1) W2 in one kernel; the other rows: SpMM + ReLU into H1, then their rows of H1 W2
            AGCN_CUDA(cudaStreamWaitEvent(s, d->ev_ready[0][0], 0));
            AGCN_CUDA(cudaEventRecord(fwd->ev[2], s));
            const float *zg = d->gathered_ptr[0];
            rc = fused_layer_async(d->indptr, d->idx, d->val, zg, fwd->w[1], fwd->z2, fwd->fused_rows, d->world == 1 ? d->per : d->n_gathered,
                                   fwd->d_status + 2, s);
            if (rc != AGCN_OK) return rc;
            SpmmLaunchPart part;
            part.unit0 = fwd->rest_unit;
            d->plan->launches_last_run = 0;
            rc = spmm_run_prepared(d->plan, d->idx, d->val, zg, 128, true, fwd->h1, 128, 128, s, AGCN_ACT_RELU, 0, part);
            if (rc != AGCN_OK) return rc;
            d->launches_last_step = d->plan->launches_last_run + 2;
            AGCN_CUDA(cudaEventRecord(d->ev_consumed[0], s));
            rc = gemm_tf32_async(fwd->h1 + fwd->fused_rows * 128, 128, fwd->w[1], fwd->z2 + fwd->fused_rows * 128, 128,
                                 d->per - fwd->fused_rows, fwd->d_status + 3, s);
            if (rc != AGCN_OK) return rc;
            AGCN_CUDA(cudaEventRecord(fwd->ev[3], s));
            h = out;
            continue;
        }
        if (rc != AGCN_OK) return rc;
        AGCN_CUDA(cudaStreamWaitEvent(s, d->ev_ready[0][0], 0));
        AGCN_CUDA(cudaEventRecord(fwd->ev[4 * layer + 2], s));          // the first slice has arrived
        rc = dist_spmm_gathered(d, 0, out, 128, AGCN_ACT_RELU, s);
        if (rc != AGCN_OK) return rc;
        AGCN_CUDA(cudaEventRecord(fwd->ev[4 * layer + 3], s));
        h = out;
    }
    return AGCN_OK;
}

// After the stream of the last run has been synchronised: the status of its GEMMs (a pipeline wait
// that ran out gives AGCN_ERR_CUDA) and, optionally, six times in milliseconds -- per layer the
// dense transform, the wait for the first slice of the exchange, and the SpMM (which includes the
// waits for later slices).
extern "C" int agcn_gcn2_forward_status(agcn_gcn2 *fwd, float *ms6)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(fwd != nullptr, "agcn_gcn2_forward_status: null argument");
    int status[4] = {0, 0, 0, 0};
    AGCN_CUDA(cudaMemcpy(status, fwd->d_status, sizeof(status), cudaMemcpyDeviceToHost));
    if (status[0] != 0 || status[1] != 0 || status[2] != 0 || status[3] != 0) {
        set_error("agcn_gcn2_forward: a pipeline wait of the dense transform ran out (layer %d); the output is incomplete",
                  status[0] != 0 ? 1 : 2);
        return AGCN_ERR_CUDA;
    }
    if (ms6 != nullptr)
        for (int layer = 0; layer < 2; layer++)
            for (int k = 0; k < 3; k++)
                AGCN_CUDA(cudaEventElapsedTime(&ms6[3 * layer + k], fwd->ev[4 * layer + k], fwd->ev[4 * layer + k + 1]));
    return AGCN_OK;
}

extern "C" int agcn_gcn2_forward_destroy(agcn_gcn2 *fwd)
{
    agcn::clear_error();
    agcn::gcn2_free(fwd);
    return AGCN_OK;
}
