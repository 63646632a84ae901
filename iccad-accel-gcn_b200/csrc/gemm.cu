// C-ABI entry point of the GCN feature transform Z = H * W (TF32 tensor cores).
// The reference has no dense transform (it benchmarks the SpMM alone); this is the X*W step of a
// GCN layer around that SpMM.
#include "host_common.h"
#include "internal.h"
#include "kernels/gemm_tf32_kernels.cuh"
#include "kernels/fused_layer_kernels.cuh"

#include <cudaTypedefs.h>
#include <mutex>

namespace agcn {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int get_encode_fn(EncodeTiledFn *out)
{
    static EncodeTiledFn cached = nullptr;
    if (cached == nullptr) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        AGCN_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess) {
            set_error("agcn_gemm_tf32: the driver does not export cuTensorMapEncodeTiled");
            return AGCN_ERR_CUDA;
        }
        cached = reinterpret_cast<EncodeTiledFn>(fn);
    }
    *out = cached;
    return AGCN_OK;
}

static const char *gemm_status_text(int status)
{
    return status == GEMM_ERR_TIMEOUT_PRODUCER ? "TMA producer" : status == GEMM_ERR_TIMEOUT_MMA ? "MMA issuer" : "epilogue";
}

// Checks the arguments, encodes the tensor map of H and launches.  Nothing is allocated and the
// stream is not synchronised; *d_status (device, zeroed here on the stream) receives a GEMM_ERR_*
// code if a pipeline wait runs out.
static int gemm_tf32_launch(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz, int64_t m_rows,
                            int k_dim, int n_dim, int *d_status, cudaStream_t s, uint32_t spin_limit, int skip_first_load)
{
    AGCN_REQUIRE(d_h != nullptr && d_w != nullptr && d_z != nullptr && d_status != nullptr, "agcn_gemm_tf32: null pointer");
    AGCN_REQUIRE(k_dim == GEMM_DIM && n_dim == GEMM_DIM,
                 "agcn_gemm_tf32: only K = N = %d is built (got K = %d, N = %d)", GEMM_DIM, k_dim, n_dim);
    AGCN_REQUIRE(m_rows >= 0 && m_rows < ((int64_t)1 << 31) * GEMM_TILE_M / 2, "agcn_gemm_tf32: row count out of range");
    AGCN_REQUIRE(ldh >= GEMM_DIM && ldz >= GEMM_DIM && ldh % 4 == 0 && ldz % 4 == 0,
                 "agcn_gemm_tf32: row strides must be >= 128 and multiples of 4 floats");
    AGCN_REQUIRE(aligned16(d_h) && aligned16(d_z), "agcn_gemm_tf32: H and Z must be 16-byte aligned");
    AGCN_CUDA(cudaMemsetAsync(d_status, 0, sizeof(int), s));
    if (m_rows == 0) return AGCN_OK;

    EncodeTiledFn encode = nullptr;
    int rc = get_encode_fn(&encode);
    if (rc != AGCN_OK) return rc;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)GEMM_DIM, (cuuint64_t)m_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ldh * 4};
    const cuuint32_t box[2] = {GEMM_KBLK, GEMM_TILE_M};
    const cuuint32_t elem[2] = {1, 1};
    CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(d_h), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        set_error("agcn_gemm_tf32: cuTensorMapEncodeTiled failed (%d)", (int)cr);
        return AGCN_ERR_CUDA;
    }

    // per-device facts, looked up once
    static int sm_count_of[64] = {};
    int dev = 0;
    AGCN_CUDA(cudaGetDevice(&dev));
    AGCN_REQUIRE(dev >= 0 && dev < 64, "agcn_gemm_tf32: device ordinal %d not supported", dev);
    if (sm_count_of[dev] == 0) {
        int sm_count = 0;
        AGCN_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
        AGCN_CUDA(cudaFuncSetAttribute(gemm_tf32_128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES));
        sm_count_of[dev] = sm_count;
    }
    const int n_tiles = (int)ceil_div(m_rows, GEMM_TILE_M);
    const int grid = n_tiles < sm_count_of[dev] ? n_tiles : sm_count_of[dev];
    gemm_tf32_128_kernel<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(map, d_w, d_z, ldz, m_rows, n_tiles, d_status, spin_limit,
                                                                      skip_first_load);
    AGCN_LAUNCH_CHECK("gemm_tf32_128_kernel");
    return AGCN_OK;
}

// status word of the synchronous entry points: one per device, allocated on first use and kept
static int gemm_status_word(int **out)
{
    static std::mutex mutex;
    static int *word_of[64] = {};
    int dev = 0;
    AGCN_CUDA(cudaGetDevice(&dev));
    AGCN_REQUIRE(dev >= 0 && dev < 64, "agcn_gemm_tf32: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lock(mutex);
    if (word_of[dev] == nullptr) AGCN_CUDA(cudaMalloc(&word_of[dev], sizeof(int)));
    *out = word_of[dev];
    return AGCN_OK;
}

static int gemm_tf32_sync(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz, int64_t m_rows,
                          int k_dim, int n_dim, cudaStream_t s, uint32_t spin_limit, int skip_first_load)
{
    int *d_status = nullptr;
    int rc = gemm_status_word(&d_status);
    if (rc != AGCN_OK) return rc;
    rc = gemm_tf32_launch(d_h, ldh, d_w, d_z, ldz, m_rows, k_dim, n_dim, d_status, s, spin_limit, skip_first_load);
    if (rc != AGCN_OK) return rc;
    int status = 0;
    AGCN_CUDA(cudaMemcpyAsync(&status, d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaStreamSynchronize(s));
    if (status != 0) {
        set_error("agcn_gemm_tf32: a pipeline wait ran out (%s); the output is incomplete", gemm_status_text(status));
        return AGCN_ERR_CUDA;
    }
    return AGCN_OK;
}

int gemm_tf32_async(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz, int64_t m_rows,
                    int *d_status, cudaStream_t s)
{
    return gemm_tf32_launch(d_h, ldh, d_w, d_z, ldz, m_rows, GEMM_DIM, GEMM_DIM, d_status, s, GEMM_SPIN_LIMIT, 0);
}

}  // namespace agcn

extern "C" int agcn_gemm_tf32(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz,
                              int64_t m_rows, int k_dim, int n_dim, void *stream)
{
    agcn::clear_error();
    return agcn::gemm_tf32_sync(d_h, ldh, d_w, d_z, ldz, m_rows, k_dim, n_dim, static_cast<cudaStream_t>(stream),
                                agcn::GEMM_SPIN_LIMIT, 0);
}

extern "C" int agcn_gemm_tf32_async(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz,
                                    int64_t m_rows, int k_dim, int n_dim, int32_t *d_status, void *stream)
{
    agcn::clear_error();
    return agcn::gemm_tf32_launch(d_h, ldh, d_w, d_z, ldz, m_rows, k_dim, n_dim, d_status, static_cast<cudaStream_t>(stream),
                                  agcn::GEMM_SPIN_LIMIT, 0);
}

extern "C" int agcn_gemm_tf32_selftest_timeout(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz,
                                               int64_t m_rows, void *stream)
{
    agcn::clear_error();
    // 4096 polls of about 100 ns: the starved wait gives up after well under a millisecond
    return agcn::gemm_tf32_sync(d_h, ldh, d_w, d_z, ldz, m_rows, agcn::GEMM_DIM, agcn::GEMM_DIM,
                                static_cast<cudaStream_t>(stream), 4096u, 1);
}

// ---------------------------------------------------------------------------
// GCN layer boundary fused into one kernel for the light rows of a degree-ordered block:
// Z2[r] = relu(A[r, :] * Z1) * W, the activations staying in shared memory between the gather and the
// tensor-core product (kernels/fused_layer_kernels.cuh).  The reference stops at the SpMM
// (spmm_accel.cu:104-108); this is the step a GCN puts behind it.
namespace agcn {

// Rows [0, m_rows) of the block must all have at most FUSED_MAX_DEG nonzeros (the caller checks: the
// kernel clamps, it does not verify).  Nothing is allocated, the stream is not synchronised;
// *d_status (device, zeroed here on the stream) receives a GEMM_ERR_* code if a pipeline wait runs out.
int fused_layer_async(const int *d_indptr, const int *d_indices, const float *d_vals, const float *d_z_in, const float *d_w,
                      float *d_z_out, int64_t m_rows, int64_t n_cols, int *d_status, cudaStream_t s)
{
    AGCN_REQUIRE(d_indptr != nullptr && d_z_in != nullptr && d_w != nullptr && d_z_out != nullptr && d_status != nullptr,
                 "agcn_gcn_fused_layer: null pointer");
    AGCN_REQUIRE(m_rows >= 0 && m_rows < ((int64_t)1 << 31) * GEMM_TILE_M / 2 && n_cols > 0, "agcn_gcn_fused_layer: row or column count out of range");
    AGCN_REQUIRE(aligned16(d_z_in) && aligned16(d_z_out), "agcn_gcn_fused_layer: Z1 and Z2 must be 16-byte aligned");
    AGCN_CUDA(cudaMemsetAsync(d_status, 0, sizeof(int), s));
    if (m_rows == 0) return AGCN_OK;
    AGCN_REQUIRE(d_indices != nullptr && d_vals != nullptr, "agcn_gcn_fused_layer: null indices or values");

    static int sm_count_of[64] = {};
    int dev = 0;
    AGCN_CUDA(cudaGetDevice(&dev));
    AGCN_REQUIRE(dev >= 0 && dev < 64, "agcn_gcn_fused_layer: device ordinal %d not supported", dev);
    if (sm_count_of[dev] == 0) {
        int sm_count = 0;
        AGCN_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
        AGCN_CUDA(cudaFuncSetAttribute(gcn_fused_layer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FUSED_SMEM_BYTES));
        sm_count_of[dev] = sm_count;
    }
    const int n_tiles = (int)ceil_div(m_rows, GEMM_TILE_M);
    const int grid = n_tiles < sm_count_of[dev] ? n_tiles : sm_count_of[dev];
    gcn_fused_layer_kernel<<<grid, FUSED_THREADS, FUSED_SMEM_BYTES, s>>>(d_indptr, d_indices, d_vals, d_z_in, d_w, d_z_out, m_rows,
                                                                         n_cols, n_tiles, d_status, GEMM_SPIN_LIMIT);
    AGCN_LAUNCH_CHECK("gcn_fused_layer_kernel");
    return AGCN_OK;
}

int fused_layer_max_degree() { return FUSED_MAX_DEG; }

}  // namespace agcn

extern "C" int agcn_gcn_fused_layer(const int32_t *d_indptr, const int32_t *d_indices, const float *d_vals, const float *d_z_in,
                                    const float *d_w, float *d_z_out, int64_t m_rows, int64_t n_cols, int32_t *d_status, void *stream)
{
    agcn::clear_error();
    return agcn::fused_layer_async(d_indptr, d_indices, d_vals, d_z_in, d_w, d_z_out, m_rows, n_cols, d_status,
                                   static_cast<cudaStream_t>(stream));
}
