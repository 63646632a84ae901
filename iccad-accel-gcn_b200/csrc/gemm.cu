// C-ABI entry point of the GCN feature transform Z = H * W (TF32 tensor cores).
// The reference has no dense transform (it benchmarks the SpMM alone); this is the X*W step of a
// GCN layer around that SpMM.
#include "host_common.h"
#include "kernels/gemm_tf32_kernels.cuh"

#include <cudaTypedefs.h>

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

static int gemm_tf32(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz, int64_t m_rows,
                     int k_dim, int n_dim, cudaStream_t s)
{
    AGCN_REQUIRE(d_h != nullptr && d_w != nullptr && d_z != nullptr, "agcn_gemm_tf32: null pointer");
    AGCN_REQUIRE(k_dim == GEMM_DIM && n_dim == GEMM_DIM,
                 "agcn_gemm_tf32: only K = N = %d is built (got K = %d, N = %d)", GEMM_DIM, k_dim, n_dim);
    AGCN_REQUIRE(m_rows >= 0 && m_rows < ((int64_t)1 << 31) * GEMM_TILE_M / 2, "agcn_gemm_tf32: row count out of range");
    AGCN_REQUIRE(ldh >= GEMM_DIM && ldz >= GEMM_DIM && ldh % 4 == 0 && ldz % 4 == 0,
                 "agcn_gemm_tf32: row strides must be >= 128 and multiples of 4 floats");
    AGCN_REQUIRE(aligned16(d_h) && aligned16(d_z), "agcn_gemm_tf32: H and Z must be 16-byte aligned");
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

    int dev = 0, sm_count = 0;
    AGCN_CUDA(cudaGetDevice(&dev));
    AGCN_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
    AGCN_CUDA(cudaFuncSetAttribute(gemm_tf32_128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES));
    DeviceScratch scratch;
    AGCN_ALLOC(d_err, scratch, int, 1);
    AGCN_CUDA(cudaMemsetAsync(d_err, 0, sizeof(int), s));
    const int n_tiles = (int)ceil_div(m_rows, GEMM_TILE_M);
    const int grid = n_tiles < sm_count ? n_tiles : sm_count;
    gemm_tf32_128_kernel<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, s>>>(map, d_w, d_z, ldz, m_rows, n_tiles, d_err);
    AGCN_LAUNCH_CHECK("gemm_tf32_128_kernel");
    int err = 0;
    AGCN_CUDA(cudaMemcpyAsync(&err, d_err, sizeof(int), cudaMemcpyDeviceToHost, s));
    AGCN_CUDA(cudaStreamSynchronize(s));
    if (err != 0) {
        set_error("agcn_gemm_tf32: a pipeline wait ran out (%s); the output is incomplete",
                  err == GEMM_ERR_TIMEOUT_PRODUCER ? "TMA producer" : err == GEMM_ERR_TIMEOUT_MMA ? "MMA issuer" : "epilogue");
        return AGCN_ERR_CUDA;
    }
    return AGCN_OK;
}

}  // namespace agcn

extern "C" int agcn_gemm_tf32(const float *d_h, int64_t ldh, const float *d_w, float *d_z, int64_t ldz,
                              int64_t m_rows, int k_dim, int n_dim, void *stream)
{
    agcn::clear_error();
    return agcn::gemm_tf32(d_h, ldh, d_w, d_z, ldz, m_rows, k_dim, n_dim, static_cast<cudaStream_t>(stream));
}
