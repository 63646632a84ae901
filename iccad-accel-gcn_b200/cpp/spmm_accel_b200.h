// The B200 SpMM as a harness plug-in: the counterpart of SPMM_ACCEL
// (spmm_accel.h:4-20), over the C ABI of libaccelgcn.so.
#pragma once
#include "spmm_plugin.h"

struct agcn_spmm_plan;

class SPMM_ACCEL_B200 : public SPMM_BASE
{
public:
    using SPMM_BASE::SPMM_BASE;
    ~SPMM_ACCEL_B200() override;

    // Where <graph>.block4 is read from on every do_test; the reference hard-codes
    // "../block_level_meta/" relative to its build directory (spmm_accel.cu:122).
    std::string meta_dir = "../block_level_meta/";
    int n_blocks = 0;

    double do_test(bool timing, int dim) override;

protected:
    void run(int dim) override;

private:
    int *block4_ = nullptr;             // device copy of the .block4 array
    agcn_spmm_plan *plan_ = nullptr;
    void release();
};
