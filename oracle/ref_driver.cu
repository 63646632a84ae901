/*
 * TEST / BENCHMARK INFRASTRUCTURE ONLY.  A thin C-ABI driver around the
 * reference's own, unmodified CUDA sources (spmm_accel.cu, spmm_cusparse.cu,
 * spmm_gnna.cu), which the Makefile compiles from where they lie in the
 * reference tree into oracle/_ref/libref_accel.so.  It exists so that the
 * reference kernel can be run on this project's inputs: as the parity oracle
 * for the SpMM, and as the kernel to beat in the benchmark.  No reference
 * source is copied here; this file only calls the reference's public classes
 * (SPMM_ACCEL, SPMM_GNNA, spmm_cusparse) the way its harness main.cu:131-167
 * does.
 *
 * The reference classes want CUDA managed memory and find their metadata by
 * a path relative to the working directory ("../block_level_meta/<graph>.block4",
 * spmm_accel.cu:122), so the driver copies the caller's host arrays into
 * managed buffers, writes the .block4 array under <workdir>/block_level_meta/
 * and changes into <workdir>/build/ for the duration of the call.
 *
 * Limits inherited from the reference (never call it outside them): dim <= 128,
 * n_rows * dim < 2^31 (int index arithmetic, spmm_accel.cu:75,84), Y zeroed
 * before the launch (rows of degree >= 33 are accumulated with atomicAdd).
 */
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unistd.h>
#include <sys/stat.h>

#include "spmm_accel.h"
#include "spmm_gnna.h"
#include "spmm_cusparse.h"

using namespace std;

string base_dir = "../graphs/";   // the reference sources declare these extern (spmm_accel.cu:9)
string graph = "ref_case";

namespace {

struct Managed {
    int *ptr = nullptr, *idx = nullptr;
    float *val = nullptr, *vin = nullptr, *vout = nullptr;
    ~Managed() { cudaFree(ptr); cudaFree(idx); cudaFree(val); cudaFree(vin); cudaFree(vout); }
};

int stage(Managed &m, const int32_t *indptr, const int32_t *idx, const float *val, const float *x,
          int64_t n_rows, int64_t nnz, int dim)
{
    if (dim < 1 || dim > 128 || n_rows * (int64_t)dim >= (int64_t)INT32_MAX) return -1;
    if (cudaMallocManaged(&m.ptr, (n_rows + 1) * sizeof(int)) != cudaSuccess) return -2;
    if (cudaMallocManaged(&m.idx, (nnz > 0 ? nnz : 1) * sizeof(int)) != cudaSuccess) return -2;
    if (cudaMallocManaged(&m.val, (nnz > 0 ? nnz : 1) * sizeof(float)) != cudaSuccess) return -2;
    if (cudaMallocManaged(&m.vin, n_rows * dim * sizeof(float)) != cudaSuccess) return -2;
    if (cudaMallocManaged(&m.vout, n_rows * dim * sizeof(float)) != cudaSuccess) return -2;
    memcpy(m.ptr, indptr, (n_rows + 1) * sizeof(int));
    memcpy(m.idx, idx, nnz * sizeof(int));
    memcpy(m.val, val, nnz * sizeof(float));
    memcpy(m.vin, x, n_rows * dim * sizeof(float));
    memset(m.vout, 0, n_rows * dim * sizeof(float));
    return 0;
}

// <workdir>/block_level_meta/ref_case.block4 + cwd = <workdir>/build
int enter_workdir(const char *workdir, const int32_t *block4, int64_t n_blocks, string &old_cwd)
{
    char buf[4096];
    if (getcwd(buf, sizeof(buf)) == nullptr) return -3;
    old_cwd = buf;
    const string w(workdir);
    mkdir((w + "/block_level_meta").c_str(), 0777);
    mkdir((w + "/build").c_str(), 0777);
    if (block4 != nullptr) {
        FILE *f = fopen((w + "/block_level_meta/" + graph + ".block4").c_str(), "wb");
        if (f == nullptr) return -3;
        fwrite(block4, 16, (size_t)n_blocks, f);
        fclose(f);
    }
    return chdir((w + "/build").c_str()) == 0 ? 0 : -3;
}

}  // namespace

extern "C" {

/* Runs the reference Accel-GCN kernel once on a zeroed Y (times == 0) and
 * copies Y back, or times it with the reference protocol (4 + 4 launches,
 * spmm_base.h:34-63) and returns mean seconds per launch in *seconds. */
int ref_accel_spmm(const char *workdir, const int32_t *block4, int64_t n_blocks,
                   const int32_t *indptr, const int32_t *idx, const float *val, const float *x, float *y,
                   int64_t n_rows, int64_t nnz, int dim, int timing, double *seconds)
{
    Managed m;
    int rc = stage(m, indptr, idx, val, x, n_rows, nnz, dim);
    if (rc != 0) return rc;
    string old_cwd;
    rc = enter_workdir(workdir, block4, n_blocks, old_cwd);
    if (rc != 0) return rc;
    {
        SPMM_ACCEL accel(graph, m.ptr, m.idx, m.val, m.vin, m.vout, (int)n_rows, (int)nnz, dim);
        const double t = accel.do_test(timing != 0, dim);
        if (seconds != nullptr) *seconds = t;
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (chdir(old_cwd.c_str()) != 0) return -3;
    if (e != cudaSuccess) return -4;
    if (y != nullptr && timing == 0) memcpy(y, m.vout, n_rows * dim * sizeof(float));
    return 0;
}

/* cusparseSpMM exactly as the reference calls it (spmm_cusparse.cu:6-62):
 * times == 0 runs once and returns Y, otherwise 10 + 10 launches timed. */
int ref_cusparse_spmm(const int32_t *indptr, const int32_t *idx, const float *val, const float *x, float *y,
                      int64_t n_rows, int64_t nnz, int dim, int timing, double *seconds)
{
    Managed m;
    int rc = stage(m, indptr, idx, val, x, n_rows, nnz, dim);
    if (rc != 0) return rc;
    const double t = spmm_cusparse(m.ptr, m.idx, m.val, m.vin, m.vout, (int)n_rows, (int)nnz, dim, timing ? 10 : 0);
    if (seconds != nullptr) *seconds = t;
    if (cudaDeviceSynchronize() != cudaSuccess) return -4;
    if (y != nullptr && timing == 0) memcpy(y, m.vout, n_rows * dim * sizeof(float));
    return 0;
}

/* GNNAdvisor kernel as the reference times it (main.cu:164-165); it ignores
 * the values of A, so it is timed only, never compared. */
int ref_gnna_time(const char *workdir, const int32_t *indptr, const int32_t *idx, const float *val, const float *x,
                  int64_t n_rows, int64_t nnz, int dim, double *seconds)
{
    Managed m;
    int rc = stage(m, indptr, idx, val, x, n_rows, nnz, dim);
    if (rc != 0) return rc;
    string old_cwd;
    rc = enter_workdir(workdir, nullptr, 0, old_cwd);
    if (rc != 0) return rc;
    {
        SPMM_GNNA gnna(graph, m.ptr, m.idx, m.val, m.vin, m.vout, (int)n_rows, (int)nnz, dim);
        const double t = gnna.do_test(true, dim);
        if (seconds != nullptr) *seconds = t;
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (chdir(old_cwd.c_str()) != 0) return -3;
    return e == cudaSuccess ? 0 : -4;
}

}  // extern "C"
