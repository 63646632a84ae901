// spmm_test -- benchmark harness with the reference's command line and output
// format (main.cu:184-222):
//
//     spmm_test <graph> <dim>     check against cuSPARSE, then time, one width
//     spmm_test                   time every ../graphs/*.config, widths 16..128
//
// run from a build directory beside graphs/ and block_level_meta/, exactly as the
// reference binary is (README.md:70-83).  It reads the degree-ordered CSR from
// ../graphs/<g>.new_indptr / .new_indices (raw int32, main.cu:62-63), fills the
// values with 1 and X with uniform(0,1) numbers from seed 123 (main.cu:90-121),
// and prints
//     CHECKING ... / err sum = ... validation pass!|fail!        (main.cu:40-49)
//     <cur>/<total> <graph> <dim> cusparse <microseconds>        (main.cu:161-167)
//     <cur>/<total> <graph> <dim> accel <microseconds>
// The GNNAdvisor line of the reference is not produced (that kernel is not part
// of this library).  Differences: device memory instead of managed memory,
// 64-bit file sizes, every CUDA call checked, and an extra "accel_event" line
// with the CUDA-event time of the same launches.
#include <cusparse.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <filesystem>
#include <fstream>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include "spmm_accel_b200.h"

namespace fs = std::filesystem;

static std::string base_dir = "../graphs/";
static int dim_min = 16, dim_max = 128, dim_step = 1;      // main.cu:12
static int total_file_cnt = 0, current_file_cnt = 0;

#define CK(call)                                                                              \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess) {                                                              \
            fprintf(stderr, "%s: %s (%s:%d)\n", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
            exit(2);                                                                          \
        }                                                                                     \
    } while (0)
#define CKS(call)                                                                             \
    do {                                                                                      \
        cusparseStatus_t s_ = (call);                                                         \
        if (s_ != CUSPARSE_STATUS_SUCCESS) {                                                  \
            fprintf(stderr, "%s: cusparse status %d (%s:%d)\n", #call, (int)s_, __FILE__, __LINE__); \
            exit(2);                                                                          \
        }                                                                                     \
    } while (0)

template <typename T>
static std::vector<T> read_raw(const std::string &path)
{
    std::ifstream in(path, std::ios::binary | std::ios::ate);
    if (!in) {
        fprintf(stderr, "cannot open %s\n", path.c_str());
        exit(2);
    }
    const int64_t bytes = in.tellg();
    std::vector<T> out((size_t)(bytes / (int64_t)sizeof(T)));
    in.seekg(0);
    in.read(reinterpret_cast<char *>(out.data()), (std::streamsize)(out.size() * sizeof(T)));
    return out;
}

template <typename T>
static T *to_device(const std::vector<T> &h)
{
    T *d = nullptr;
    CK(cudaMalloc(&d, std::max<size_t>(h.size(), 1) * sizeof(T)));
    CK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
    return d;
}

// cusparseSpMM as the reference calls it (spmm_cusparse.cu:6-62): CSR, row-major dense,
// alpha = 1, beta = 0, default algorithm; times == 0 runs once, otherwise 10 + 10 launches.
static double spmm_cusparse(int *ptr, int *idx, float *val, float *vin, float *vout, int num_v, int num_e, int dim, int times)
{
    cusparseHandle_t handle;
    cusparseSpMatDescr_t a;
    cusparseDnMatDescr_t b, c;
    const float alpha = 1.f, beta = 0.f;
    CKS(cusparseCreate(&handle));
    CKS(cusparseCreateCsr(&a, num_v, num_v, num_e, ptr, idx, val, CUSPARSE_INDEX_32I, CUSPARSE_INDEX_32I,
                          CUSPARSE_INDEX_BASE_ZERO, CUDA_R_32F));
    CKS(cusparseCreateDnMat(&b, num_v, dim, dim, vin, CUDA_R_32F, CUSPARSE_ORDER_ROW));
    CKS(cusparseCreateDnMat(&c, num_v, dim, dim, vout, CUDA_R_32F, CUSPARSE_ORDER_ROW));
    size_t buf_bytes = 0;
    CKS(cusparseSpMM_bufferSize(handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, a, b,
                                &beta, c, CUDA_R_32F, CUSPARSE_SPMM_ALG_DEFAULT, &buf_bytes));
    void *buf = nullptr;
    CK(cudaMalloc(&buf, std::max<size_t>(buf_bytes, 16)));
    auto once = [&]() {
        CKS(cusparseSpMM(handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, a, b, &beta, c,
                         CUDA_R_32F, CUSPARSE_SPMM_ALG_DEFAULT, buf));
    };
    double seconds = 0.0;
    if (times == 0) {
        once();
        CK(cudaDeviceSynchronize());
    } else {
        const int reps = 10;
        for (int i = 0; i < reps; i++) once();
        CK(cudaDeviceSynchronize());
        for (int i = 0; i < reps; i++) {
            const auto t0 = std::chrono::steady_clock::now();
            once();
            CK(cudaDeviceSynchronize());
            seconds += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        }
        seconds /= reps;
    }
    cusparseDestroySpMat(a);
    cusparseDestroyDnMat(b);
    cusparseDestroyDnMat(c);
    cusparseDestroy(handle);
    cudaFree(buf);
    return seconds;
}

// mean absolute error below 1e-3 passes; the first element off by more than 0.1 is reported (main.cu:18-51)
static bool check_err(const std::vector<float> &out, const std::vector<float> &ref)
{
    double err_sum = 0.0;
    bool reported = false;
    for (size_t i = 0; i < out.size(); i++) {
        const double err = std::fabs((double)out[i] - (double)ref[i]);
        err_sum += err;
        if (!(err <= 0.1) && !reported) {
            reported = true;
            std::cout << "err at " << i << std::endl;
        }
    }
    const bool pass = out.empty() || err_sum / (double)out.size() < 0.001;
    std::cout << "err sum = " << err_sum << "  " << (pass ? "validation pass!" : "validation fail!") << std::endl;
    return pass;
}

static bool test_graph(const std::string &graph, int spec_dim, bool checking, bool timing)
{
    int lo = dim_min, hi = dim_max;
    if (spec_dim > 0) lo = hi = spec_dim;

    const std::vector<int> indptr = read_raw<int>(base_dir + graph + ".new_indptr");
    const std::vector<int> indices = read_raw<int>(base_dir + graph + ".new_indices");
    const int v_num = (int)indptr.size() - 1, e_num = (int)indices.size();
    if (v_num <= 0) {
        fprintf(stderr, "%s: empty graph\n", graph.c_str());
        return false;
    }
    const size_t dense = (size_t)v_num * (size_t)hi;
    std::vector<float> val((size_t)e_num, 1.0f), vin(dense);      // value mode 3 of main.cu:113-121
    std::default_random_engine engine;
    engine.seed(123);
    std::uniform_real_distribution<float> rd(0, 1);
    std::generate(vin.begin(), vin.end(), [&]() { return rd(engine); });

    int *d_ptr = to_device(indptr), *d_idx = to_device(indices);
    float *d_val = to_device(val), *d_vin = to_device(vin), *d_out = nullptr, *d_ref = nullptr;
    CK(cudaMalloc(&d_out, dense * sizeof(float)));
    CK(cudaMalloc(&d_ref, dense * sizeof(float)));
    CK(cudaMemset(d_out, 0xff, dense * sizeof(float)));           // NaN pattern: the plug-in must overwrite all of it

    SPMM_ACCEL_B200 accel(graph, d_ptr, d_idx, d_val, d_vin, d_out, v_num, e_num, hi);
    bool all_pass = true;
    for (int dim = lo; dim <= hi; dim += dim_step) {
        if (checking) {
            std::cout << "CHECKING ..." << std::endl;
            spmm_cusparse(d_ptr, d_idx, d_val, d_vin, d_ref, v_num, e_num, dim, 0);
            if (accel.do_test(false, dim) < 0) return false;
            std::vector<float> out((size_t)v_num * dim), ref((size_t)v_num * dim);
            CK(cudaMemcpy(out.data(), d_out, out.size() * sizeof(float), cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(ref.data(), d_ref, ref.size() * sizeof(float), cudaMemcpyDeviceToHost));
            std::cout << "checking accel" << std::endl;
            all_pass = check_err(out, ref) && all_pass;
        }
        if (timing) {
            std::cout << "TIMING ..." << std::endl;
            const std::string tag = std::to_string(current_file_cnt) + "/" + std::to_string(total_file_cnt) + " " + graph +
                                    " " + std::to_string(dim);
            const double t_cusparse = spmm_cusparse(d_ptr, d_idx, d_val, d_vin, d_ref, v_num, e_num, dim, 10);
            std::cout << tag << " cusparse " << t_cusparse * 1e6 << std::endl;
            const double t_accel = accel.do_test(true, dim);
            if (t_accel < 0) return false;
            std::cout << tag << " accel " << t_accel * 1e6 << std::endl;
            std::cout << tag << " accel_event " << accel.last_event_seconds() * 1e6 << std::endl;
        }
    }
    cudaFree(d_ptr); cudaFree(d_idx); cudaFree(d_val); cudaFree(d_vin); cudaFree(d_out); cudaFree(d_ref);
    return all_pass;
}

int main(int argc, char *argv[])
{
    if (argc > 2) {                                   // spmm_test artist 60
        std::cout << "dir = " << base_dir << std::endl;
        return test_graph(argv[1], atoi(argv[2]), true, true) ? 0 : 1;
    }
    std::vector<std::string> graphs;                  // spmm_test: every graph, every width
    for (const auto &f : fs::directory_iterator(base_dir))
        if (f.path().extension() == ".config") graphs.push_back(f.path().stem().string());
    std::sort(graphs.begin(), graphs.end());
    total_file_cnt = (int)graphs.size();
    for (const auto &g : graphs) {
        current_file_cnt++;
        // the reference's sweep only times (main.cu:216); AGCN_TEST_CHECK_ALL=1 also checks every width
        if (!test_graph(g, 0, getenv("AGCN_TEST_CHECK_ALL") != nullptr, true)) return 1;
        CK(cudaDeviceSynchronize());
    }
    return 0;
}
