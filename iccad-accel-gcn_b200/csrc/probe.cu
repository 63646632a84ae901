// Measurement aid: how fast can this GPU gather whole rows of a dense table that stays in L2?
// The SpMM (spmm_accel.cu:55-78 in the reference) moves nnz * dim * 4 bytes of X through the
// L2 -> SM path for 4 * dim * N bytes from HBM, so on dense graphs its ceiling is this gather rate,
// not the HBM bandwidth.  The probe issues the same access shape as the SpMM's float4 mode -- a
// slot of dim/4 lanes reads one row with 16-byte loads, four independent rows in flight per lane,
// 256 threads per block at a residency the caller chooses, the same L2 policy -- with row numbers
// from a counter-based hash instead of a column array and a plain add instead of the FMA, so what
// it measures is the memory path alone.
#include "host_common.h"
#include "kernels/primitives.cuh"
#include "kernels/ptx.cuh"

namespace agcn {

// row number of the k-th gather of a warp: multiplicative (Fibonacci) hashing, one multiply and one
// shift, so that the probe spends its instructions on loads (the table has a power-of-two row count)
__device__ __forceinline__ uint32_t probe_row(uint32_t k, int shift) { return (k * 0x9E3779B1u) >> shift; }

template <int S>
__global__ void __launch_bounds__(256)
probe_gather_kernel(const float *__restrict__ table, int row_shift, int row_floats, int rows_per_warp, float *__restrict__ sink)
{
    constexpr int NS = 32 / S;
    const int lane = lane_id(), slot = lane / S, col = (lane % S) * 4;
    const uint32_t warp = blockIdx.x * (blockDim.x >> 5) + warp_id();
    const L2Policies pol = make_l2_policies();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float *base = table + col;
    for (int i = slot; i + 3 * NS < rows_per_warp; i += 4 * NS) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const uint32_t r = probe_row(warp * (uint32_t)rows_per_warp + (uint32_t)(i + u * NS), row_shift);
            v[u] = ld_x4(base + (int64_t)r * row_floats, pol.keep);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
    }
    const float t = acc.x + acc.y + acc.z + acc.w;
    if (t == 123456.789f) sink[warp] = t;       // never true for the zero-filled table: keeps the loads alive
}

}  // namespace agcn

// table_rows (a power of two) rows of row_floats floats (32, 64 or 128: 128 / 256 / 512-byte rows); total_rows rows
// are gathered per launch; the rate over `iters` launches (after one warm-up) is returned in GB/s.
extern "C" int agcn_probe_gather_bandwidth(int64_t table_rows, int row_floats, int64_t total_rows, int iters,
                                           int resident_blocks, double *gb_per_s)
{
    using namespace agcn;
    clear_error();
    AGCN_REQUIRE(gb_per_s != nullptr, "agcn_probe_gather_bandwidth: null result pointer");
    AGCN_REQUIRE(row_floats == 32 || row_floats == 64 || row_floats == 128, "agcn_probe_gather_bandwidth: row_floats must be 32, 64 or 128");
    AGCN_REQUIRE(table_rows >= 2 && table_rows <= ((int64_t)1 << 30) && (table_rows & (table_rows - 1)) == 0 && total_rows > 0 && iters >= 1,
                 "agcn_probe_gather_bandwidth: table_rows must be a power of two, 2..2^30");
    int row_shift = 32;
    while (((int64_t)1 << (32 - row_shift)) < table_rows) row_shift--;
    AGCN_REQUIRE(resident_blocks >= 0 && resident_blocks <= 8, "agcn_probe_gather_bandwidth: resident_blocks must be 0..8");
    const int rows_per_warp = 512;       // short warps, many of them: the grid must fill every SM several times over
    const int64_t warps = ceil_div(total_rows, rows_per_warp);
    AGCN_REQUIRE(warps / 8 + 1 < ((int64_t)1 << 31), "agcn_probe_gather_bandwidth: too many rows per launch");
    const unsigned grid = (unsigned)ceil_div(warps, 8);
    DeviceScratch scratch;
    AGCN_ALLOC(table, scratch, float, table_rows * row_floats);
    AGCN_ALLOC(sink, scratch, float, (int64_t)grid * 8);
    AGCN_CUDA(cudaMemset(table, 0, (size_t)table_rows * row_floats * sizeof(float)));
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    AGCN_CUDA(cudaEventCreate(&e0));
    AGCN_CUDA(cudaEventCreate(&e1));
    // resident_blocks > 0: unused dynamic shared memory sized so that only that many thread blocks fit
    // on an SM (the SpMM keeps 5); 0 = whatever the registers allow
    const size_t smem = resident_blocks == 0 ? 0 : (size_t)(220 * 1024 / resident_blocks) & ~(size_t)1023;
    if (smem > 48 * 1024) {
        AGCN_CUDA(cudaFuncSetAttribute(probe_gather_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        AGCN_CUDA(cudaFuncSetAttribute(probe_gather_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        AGCN_CUDA(cudaFuncSetAttribute(probe_gather_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    auto launch = [&]() {
        if (row_floats == 32) probe_gather_kernel<8><<<grid, 256, smem>>>(table, row_shift, row_floats, rows_per_warp, sink);
        else if (row_floats == 64) probe_gather_kernel<16><<<grid, 256, smem>>>(table, row_shift, row_floats, rows_per_warp, sink);
        else probe_gather_kernel<32><<<grid, 256, smem>>>(table, row_shift, row_floats, rows_per_warp, sink);
    };
    launch();                                             // warm-up: brings the table into L2
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaEventRecord(e0);
    for (int i = 0; i < iters && e == cudaSuccess; i++) launch();
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaEventRecord(e1);
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) {
        set_error("agcn_probe_gather_bandwidth: %s", cudaGetErrorString(e));
        return AGCN_ERR_CUDA;
    }
    // every warp gathers rows_per_warp rows (rounded down to whole batches of four per slot)
    const int ns = 32 / (row_floats / 4);
    const int64_t per_warp = (int64_t)(rows_per_warp / (4 * ns)) * (4 * ns);
    *gb_per_s = (double)warps * (double)per_warp * row_floats * 4.0 * iters / ((double)ms * 1e-3) / 1e9;
    return AGCN_OK;
}
