"""Host-side Python mirror of the Accel-GCN hot-path interfaces, over the C ABI
of libaccelgcn.so (include/accelgcn.h).

    partition   -- block_level_partition.py replacement (ctypes, .block4 output)
    degree_sort -- the degree ordering the reference assumes of its inputs
    spmm        -- SPMM_ACCEL plug-in mirror (do_test / run) and a functional call
    graphio     -- the reference's raw-binary graph and .block4 files
    synth       -- seeded synthetic graphs for tests and benchmarks
    sharded     -- 1D row-sharded multi-GPU SpMM (agcn_dist_*: layout, NCCL exchange and kernels in the library)
    gcn         -- two-layer GCN forward on the row blocks (agcn_gcn2_forward_*)
    gemm        -- dense feature transform on the tensor cores (agcn_gemm_tf32*)

PyTorch appears here only as the owner of device memory and streams (and of the
process group in `sharded`); all compute is in the shared library.
"""
from ._lib import AccelGcnError, load, lib_path  # noqa: F401
