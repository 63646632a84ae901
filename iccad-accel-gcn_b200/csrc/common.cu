// Error reporting and the device-wide prefix sums of the C-ABI library.
#include "host_common.h"
#include "kernels/primitives.cuh"

#include <string>

namespace agcn {

static thread_local std::string g_last_error;

void set_error(const char *fmt, ...)
{
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
}

void clear_error() { g_last_error.clear(); }

int64_t scan_tiles(int64_t n) { return ceil_div(n > 0 ? n : 1, SCAN_TILE); }

template <typename TIn, typename TAcc, typename TOut>
static int exclusive_scan(const TIn *in, TOut *out, int64_t n, TAcc *tile_sums, TAcc *total_out, cudaStream_t s)
{
    if (n <= 0) {
        if (total_out != nullptr) AGCN_CUDA(cudaMemsetAsync(total_out, 0, sizeof(TAcc), s));
        return AGCN_OK;
    }
    const int64_t tiles = scan_tiles(n);
    auto k_reduce = scan_tile_reduce_kernel<TIn, TAcc>;
    auto k_top = single_block_scan_exclusive_kernel<TAcc, OpAdd>;
    auto k_down = scan_tile_downsweep_kernel<TIn, TAcc, TOut>;
    AGCN_KERNEL(k_reduce, (unsigned)tiles, SCAN_BLOCK, s, in, n, tile_sums);
    AGCN_LAUNCH_CHECK("scan_tile_reduce_kernel");
    AGCN_KERNEL(k_top, 1, 1024, s, tile_sums, tiles, (TAcc)0, total_out);
    AGCN_LAUNCH_CHECK("single_block_scan_exclusive_kernel");
    AGCN_KERNEL(k_down, (unsigned)tiles, SCAN_BLOCK, s, in, n, (const TAcc *)tile_sums, out);
    AGCN_LAUNCH_CHECK("scan_tile_downsweep_kernel");
    return AGCN_OK;
}

int exclusive_scan_i32_i64(const int *in, int64_t *out, int64_t n, int64_t *tile_sums, int64_t *total_out, cudaStream_t s)
{
    return exclusive_scan<int, int64_t, int64_t>(in, out, n, tile_sums, total_out, s);
}
int exclusive_scan_u32_u32(const unsigned *in, unsigned *out, int64_t n, unsigned *tile_sums, cudaStream_t s)
{
    return exclusive_scan<unsigned, unsigned, unsigned>(in, out, n, tile_sums, (unsigned *)nullptr, s);
}
int exclusive_scan_u32_i32(const unsigned *in, int *out, int64_t n, int *tile_sums, cudaStream_t s)
{
    return exclusive_scan<unsigned, int, int>(in, out, n, tile_sums, (int *)nullptr, s);
}

}  // namespace agcn

extern "C" const char *agcn_last_error(void) { return agcn::g_last_error.c_str(); }
extern "C" int agcn_version(void) { return 100; }
