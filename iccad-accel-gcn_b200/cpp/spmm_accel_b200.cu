#include "spmm_accel_b200.h"

#include <cstdio>
#include <fstream>
#include <vector>

#include "../../include/accelgcn.h"

SPMM_ACCEL_B200::~SPMM_ACCEL_B200() { release(); }

void SPMM_ACCEL_B200::release()
{
    if (plan_ != nullptr) agcn_spmm_destroy(plan_);
    plan_ = nullptr;
    cudaFree(block4_);
    block4_ = nullptr;
}

// one asynchronous launch sequence on the default stream, no synchronisation (spmm_accel.cu:104-108)
void SPMM_ACCEL_B200::run(int cur_dim)
{
    if (agcn_spmm_run(plan_, idx, val, vin, cur_dim, vout, cur_dim, cur_dim, nullptr) != AGCN_OK)
        fprintf(stderr, "SPMM_ACCEL_B200::run: %s\n", agcn_last_error());
}

// load <graph>.block4, build the plan, run or time, release (spmm_accel.cu:110-139)
double SPMM_ACCEL_B200::do_test(bool timing, int cur_dim)
{
    release();
    const std::string path = meta_dir + _graph + ".block4";
    std::ifstream in(path, std::ios::binary | std::ios::ate);
    if (!in) {
        fprintf(stderr, "SPMM_ACCEL_B200: cannot open %s\n", path.c_str());
        return -1.0;
    }
    const long long bytes = in.tellg();
    if (bytes % 16 != 0) {
        fprintf(stderr, "SPMM_ACCEL_B200: %s is not a whole number of 4-tuples\n", path.c_str());
        return -1.0;
    }
    std::vector<int> host((size_t)(bytes / 4));
    in.seekg(0);
    in.read(reinterpret_cast<char *>(host.data()), bytes);
    n_blocks = (int)(bytes / 16);
    if (cudaMalloc(&block4_, bytes > 0 ? (size_t)bytes : 16) != cudaSuccess ||
        cudaMemcpy(block4_, host.data(), (size_t)bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
        fprintf(stderr, "SPMM_ACCEL_B200: device copy of %s failed\n", path.c_str());
        return -1.0;
    }
    if (agcn_spmm_create(&plan_, block4_, n_blocks, idx, num_v, num_v, num_e, nullptr) != AGCN_OK) {
        fprintf(stderr, "SPMM_ACCEL_B200: %s\n", agcn_last_error());
        release();
        return -1.0;
    }
    const double seconds = timing_body(timing, cur_dim);
    release();
    return seconds;
}
