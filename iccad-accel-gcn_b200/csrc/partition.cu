// C-ABI entry points of the block-level partitioner
// (replaces block_level_partition.py:38-106).
#include "host_common.h"
#include "internal.h"
#include "kernels/partition_kernels.cuh"

#include <cstddef>
#include <mutex>

namespace agcn {

// Tile scratch of one partitioner call: one run-head index and one tuple count per PART_TILE rows,
// the tuple total and an error word.  The regular entry point allocates it per call; the
// allocation-free one points it at a fixed array in the library's device image.
struct PartScratch {
    int *tile_head;
    int64_t *tile_count;
    int64_t *total;
    int *err;
};

// The pipeline both entry points run.  `who` names the entry point in error messages.
static int partition_pipeline(const char *who, const int *d_indptr, int64_t n_rows, int *d_block4, int64_t cap_blocks,
                              int64_t *n_blocks, const PartScratch &sc, cudaStream_t s)
{
    const int64_t tiles = ceil_div(n_rows, PART_TILE);
    AGCN_CUDA(cudaMemsetAsync(sc.err, 0, sizeof(int), s));      // the one word that must start at zero
    auto k_scan_max = single_block_scan_exclusive_kernel<int, OpMax>;
    auto k_scan_add = single_block_scan_exclusive_kernel<int64_t, OpAdd>;
    AGCN_KERNEL(part_run_heads_kernel, (unsigned)tiles, PART_BLOCK, s, d_indptr, n_rows, sc.tile_head, sc.err);
    AGCN_LAUNCH_CHECK("part_run_heads_kernel");
    AGCN_KERNEL(k_scan_max, 1, 1024, s, sc.tile_head, tiles, -1, (int *)nullptr);
    AGCN_LAUNCH_CHECK("single_block_scan_exclusive_kernel<max>");
    AGCN_KERNEL(part_count_kernel, (unsigned)tiles, PART_BLOCK, s, d_indptr, n_rows, (const int *)sc.tile_head, sc.tile_count);
    AGCN_LAUNCH_CHECK("part_count_kernel");
    AGCN_KERNEL(k_scan_add, 1, 1024, s, sc.tile_count, tiles, (int64_t)0, sc.total);
    AGCN_LAUNCH_CHECK("single_block_scan_exclusive_kernel<add>");

    int64_t total = 0;
    int err = 0;
    AGCN_CUDA(cudaMemcpyAsync(&total, sc.total, sizeof(total), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaMemcpyAsync(&err, sc.err, sizeof(err), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaStreamSynchronize(s));
    if (err != 0) {
        set_error("%s: indptr decreases somewhere (negative degree); "
                  "the reference script prints 'cur_degree number is wrong' and stops", who);
        return AGCN_ERR_RANGE;
    }
    *n_blocks = total;
    if (d_block4 == nullptr || cap_blocks == 0) return AGCN_OK;
    if (cap_blocks < total) {
        set_error("%s: %lld blocks needed, capacity %lld", who, (long long)total, (long long)cap_blocks);
        return AGCN_ERR_CAPACITY;
    }
    if (total > 0) {
        AGCN_KERNEL(part_emit_kernel, (unsigned)tiles, PART_BLOCK, s, d_indptr, n_rows, (const int *)sc.tile_head,
                    (const int64_t *)sc.tile_count, reinterpret_cast<int4 *>(d_block4));
        AGCN_LAUNCH_CHECK("part_emit_kernel");
    }
    AGCN_CUDA(cudaStreamSynchronize(s));
    return AGCN_OK;
}

int partition_device(const int *d_indptr, int64_t n_rows, int *d_block4, int64_t cap_blocks,
                     int64_t *n_blocks, cudaStream_t s)
{
    AGCN_REQUIRE(d_indptr != nullptr && n_blocks != nullptr, "agcn_partition: null pointer");
    AGCN_REQUIRE(n_rows > 0, "agcn_partition: empty graph (n_rows = %lld); the reference script raises IndexError here",
                 (long long)n_rows);
    AGCN_REQUIRE(n_rows < (int64_t)INT32_MAX, "agcn_partition: n_rows = %lld does not fit the int32 row ids of .block4",
                 (long long)n_rows);
    AGCN_REQUIRE(d_block4 == nullptr || aligned16(d_block4), "agcn_partition: block4 output must be 16-byte aligned");
    *n_blocks = 0;

    const int64_t tiles = ceil_div(n_rows, PART_TILE);
    DeviceScratch scratch;
    PartScratch sc;
    AGCN_ALLOC(tile_head, scratch, int, tiles);
    AGCN_ALLOC(tile_count, scratch, int64_t, tiles);
    AGCN_ALLOC(d_total, scratch, int64_t, 1);
    AGCN_ALLOC(d_err, scratch, int, 1);
    sc.tile_head = tile_head; sc.tile_count = tile_count; sc.total = d_total; sc.err = d_err;
    return partition_pipeline("agcn_partition", d_indptr, n_rows, d_block4, cap_blocks, n_blocks, sc, s);
}

}  // namespace agcn

extern "C" int agcn_partition_device(const int32_t *d_indptr, int64_t n_rows, int32_t *d_block4,
                                     int64_t cap_blocks, int64_t *n_blocks, void *stream)
{
    agcn::clear_error();
    return agcn::partition_device(d_indptr, n_rows, d_block4, cap_blocks, n_blocks, static_cast<cudaStream_t>(stream));
}

extern "C" int agcn_partition_host(const int32_t *h_indptr, int64_t n_rows, int32_t *h_block4,
                                   int64_t cap_blocks, int64_t *n_blocks)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(h_indptr != nullptr && n_blocks != nullptr, "agcn_partition_host: null pointer");
    AGCN_REQUIRE(n_rows > 0, "agcn_partition_host: empty graph (n_rows = %lld); the reference script raises IndexError here",
                 (long long)n_rows);
    DeviceScratch scratch;
    AGCN_ALLOC(d_indptr, scratch, int, n_rows + 1);
    AGCN_CUDA(cudaMemcpy(d_indptr, h_indptr, (size_t)(n_rows + 1) * sizeof(int), cudaMemcpyHostToDevice));
    int rc = partition_device(d_indptr, n_rows, nullptr, 0, n_blocks, nullptr);
    if (rc != AGCN_OK || h_block4 == nullptr || cap_blocks == 0) return rc;
    if (cap_blocks < *n_blocks) {
        set_error("agcn_partition_host: %lld blocks needed, capacity %lld", (long long)*n_blocks, (long long)cap_blocks);
        return AGCN_ERR_CAPACITY;
    }
    if (*n_blocks == 0) return AGCN_OK;
    AGCN_ALLOC(d_block4, scratch, int, *n_blocks * 4);
    rc = partition_device(d_indptr, n_rows, d_block4, *n_blocks, n_blocks, nullptr);
    if (rc != AGCN_OK) return rc;
    AGCN_CUDA(cudaMemcpy(h_block4, d_block4, (size_t)*n_blocks * 16, cudaMemcpyDeviceToHost));
    return AGCN_OK;
}

// ---------------------------------------------------------------------------
// Partitioner for callers that must not allocate device memory.
//
// Some hosts of this library cannot let it call cudaMalloc: a process whose
// framework allocator has already claimed all of HBM (a raw cudaMalloc then
// fails or steals from its pool), a latency-critical loop that cannot afford
// the device-wide synchronisation cudaMalloc / cudaFree imply, or a plug-in
// host that forbids allocation calls after start-up.  For them the tile
// scratch of the partitioner (one run-head index and one tuple count per 2048
// rows, plus the total and an error word) lives in a fixed array in the
// library's device image instead of a per-call allocation.  Every GPU that
// loads the library holds that array (about 96 KB) until the process exits,
// which is why it is sized for AGCN_PARTITION_NOALLOC_MAX_ROWS rows and no
// more.
//
// The array's name is only a host-side handle; its device address is looked
// up once per device with cudaGetSymbolAddress, on the first call made with
// that device current.  That first call should therefore happen before any
// stream capture is started.  All calls on a device share the array and it
// keeps what the previous call left: the error word is cleared at the start
// of every call, everything else is overwritten before it is read.  Two calls
// that overlap on the same GPU (different streams or threads) race on it.
// ---------------------------------------------------------------------------
namespace agcn {

constexpr int64_t PART_NOALLOC_MAX_ROWS = AGCN_PARTITION_NOALLOC_MAX_ROWS;
constexpr int64_t PART_NOALLOC_MAX_TILES = (PART_NOALLOC_MAX_ROWS + PART_TILE - 1) / PART_TILE;
constexpr int PART_NOALLOC_MAX_DEVICES = 64;

struct PartStaticScratch {
    int64_t tile_count[PART_NOALLOC_MAX_TILES];
    int64_t total;
    int tile_head[PART_NOALLOC_MAX_TILES];
    int err;
};

}  // namespace agcn

static __device__ __align__(256) unsigned char g_part_static_scratch[sizeof(agcn::PartStaticScratch)];

namespace agcn {

static std::mutex g_part_static_mutex;
static PartStaticScratch *g_part_static_addr[PART_NOALLOC_MAX_DEVICES] = {};

// device address of the static scratch on the current device (looked up once per device)
static int part_static_scratch(PartStaticScratch **out)
{
    int dev = -1;
    AGCN_CUDA(cudaGetDevice(&dev));
    AGCN_REQUIRE(dev >= 0 && dev < PART_NOALLOC_MAX_DEVICES, "agcn_partition_device_noalloc: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_part_static_mutex);
    if (g_part_static_addr[dev] == nullptr) {
        PartStaticScratch *ptr = nullptr;
        AGCN_CUDA(cudaGetSymbolAddress((void **)&ptr, g_part_static_scratch));
        AGCN_REQUIRE(ptr != nullptr, "agcn_partition_device_noalloc: cudaGetSymbolAddress returned a null address");
        g_part_static_addr[dev] = ptr;
    }
    *out = g_part_static_addr[dev];
    return AGCN_OK;
}

static int partition_device_noalloc(const int *d_indptr, int64_t n_rows, int *d_block4, int64_t cap_blocks,
                                    int64_t *n_blocks, cudaStream_t s)
{
    AGCN_REQUIRE(d_indptr != nullptr && n_blocks != nullptr, "agcn_partition_device_noalloc: null pointer");
    AGCN_REQUIRE(n_rows > 0, "agcn_partition_device_noalloc: empty graph (n_rows = %lld)", (long long)n_rows);
    AGCN_REQUIRE(n_rows <= PART_NOALLOC_MAX_ROWS,
                 "agcn_partition_device_noalloc: n_rows = %lld exceeds the %lld rows the static scratch is sized for; "
                 "use agcn_partition_device for larger graphs", (long long)n_rows, (long long)PART_NOALLOC_MAX_ROWS);
    AGCN_REQUIRE(d_block4 == nullptr || aligned16(d_block4), "agcn_partition_device_noalloc: block4 output must be 16-byte aligned");
    *n_blocks = 0;

    PartStaticScratch *st = nullptr;
    int rc = part_static_scratch(&st);
    if (rc != AGCN_OK) return rc;
    // st is a device address: form member addresses by arithmetic only, never dereference it here
    unsigned char *base = reinterpret_cast<unsigned char *>(st);
    PartScratch sc;
    sc.tile_count = reinterpret_cast<int64_t *>(base + offsetof(PartStaticScratch, tile_count));
    sc.total = reinterpret_cast<int64_t *>(base + offsetof(PartStaticScratch, total));
    sc.tile_head = reinterpret_cast<int *>(base + offsetof(PartStaticScratch, tile_head));
    sc.err = reinterpret_cast<int *>(base + offsetof(PartStaticScratch, err));
    return partition_pipeline("agcn_partition_device_noalloc", d_indptr, n_rows, d_block4, cap_blocks, n_blocks, sc, s);
}

}  // namespace agcn

extern "C" int agcn_partition_device_noalloc(const int32_t *d_indptr, int64_t n_rows, int32_t *d_block4,
                                             int64_t cap_blocks, int64_t *n_blocks, void *stream)
{
    agcn::clear_error();
    return agcn::partition_device_noalloc(d_indptr, n_rows, d_block4, cap_blocks, n_blocks,
                                          static_cast<cudaStream_t>(stream));
}
