// Plug-in interface of the SpMM benchmark harness, source-compatible with the
// reference's SPMM_BASE (spmm_base.h:6-65): a kernel plug-in derives from
// SPMM_BASE, inherits the constructor (borrowed pointers: row pointers, column
// ids, values, dense input, dense output; vertex / edge counts; buffer width),
// and implements
//     double do_test(bool timing, int dim);   // prepare, then run once or time
//     void   run(int dim);                    // one asynchronous launch
// timing_body() keeps the reference's protocol -- 4 warm-up launches, then 4
// launches each followed by a device synchronisation, mean host wall-clock
// seconds (spmm_base.h:34-63) -- so numbers printed by a harness built on it
// compare like for like with the reference's.  In addition every timed launch
// is bracketed by CUDA events; last_event_seconds() gives the mean device time.
#pragma once
#include <cuda_runtime.h>

#include <chrono>
#include <string>

class SPMM_BASE
{
public:
    SPMM_BASE(std::string graph_name, int *row_ptr, int *col_idx, float *values, float *dense_in, float *dense_out,
              int n_vertices, int n_edges, int width)
        : _graph(std::move(graph_name)), ptr(row_ptr), idx(col_idx), val(values), vin(dense_in), vout(dense_out),
          num_v(n_vertices), num_e(n_edges), dim(width)
    {
    }
    virtual ~SPMM_BASE() = default;

    virtual double do_test(bool timing, int dim) = 0;

    double last_event_seconds() const { return event_seconds_; }

protected:
    std::string _graph;
    int *ptr, *idx;
    float *val, *vin, *vout;
    int num_v, num_e, dim;
    dim3 grid, block;

    virtual void run(int dim) = 0;

    static constexpr int kRepeats = 4;   // spmm_base.h:44

    double timing_body(bool timing, int cur_dim)
    {
        event_seconds_ = 0.0;
        if (!timing) {
            run(cur_dim);
            cudaDeviceSynchronize();
            return 0.0;
        }
        for (int i = 0; i < kRepeats; i++) run(cur_dim);
        cudaDeviceSynchronize();
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        double wall = 0.0, dev = 0.0;
        for (int i = 0; i < kRepeats; i++) {
            const auto t0 = std::chrono::steady_clock::now();
            cudaEventRecord(e0);
            run(cur_dim);
            cudaEventRecord(e1);
            cudaDeviceSynchronize();
            wall += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            float ms = 0.f;
            cudaEventElapsedTime(&ms, e0, e1);
            dev += ms * 1e-3;
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        event_seconds_ = dev / kRepeats;
        return wall / kRepeats;
    }

private:
    double event_seconds_ = 0.0;
};
