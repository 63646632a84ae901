"""Builds lib/libaccelgcn.so from csrc/ with nvcc for sm_100a (cross-compiles without a GPU).

    python iccad-accel-gcn_b200/build.py [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["common.cu", "partition.cu", "degree_sort.cu", "spmm.cu", "spmm_tiled.cu", "host_spmm.cu", "gemm.cu", "layout.cu", "dist.cu", "probe.cu"]
LIB = os.path.join(HERE, "lib", "libaccelgcn.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def _inputs():
    files = [os.path.join(HERE, "csrc", s) for s in SOURCES]
    files.append(os.path.join(HERE, "..", "include", "accelgcn.h"))
    for root, _dirs, names in os.walk(os.path.join(HERE, "csrc")):
        files += [os.path.join(root, n) for n in names if n.endswith((".cuh", ".h"))]
    return files


HARNESS = os.path.join(HERE, "lib", "spmm_test")
HARNESS_SOURCES = ["spmm_test.cu", "spmm_accel_b200.cu"]


def build_harness(force: bool = False) -> str:
    """lib/spmm_test: the reference-compatible benchmark harness (cpp/), linked against the library."""
    build()
    srcs = [os.path.join(HERE, "cpp", s) for s in HARNESS_SOURCES]
    deps = srcs + [os.path.join(HERE, "cpp", h) for h in ("spmm_plugin.h", "spmm_accel_b200.h")] + [LIB]
    if not force and os.path.exists(HARNESS) and all(os.path.getmtime(f) <= os.path.getmtime(HARNESS) for f in deps):
        return HARNESS
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-o", HARNESS, *srcs,
           "-L" + os.path.dirname(LIB), "-laccelgcn", "-lcusparse", "-Xlinker", "-rpath=$ORIGIN"]
    subprocess.check_call(cmd)
    return HARNESS


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(LIB) and all(os.path.getmtime(f) <= os.path.getmtime(LIB) for f in _inputs()):
        return LIB
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    cmd = ["nvcc", *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", LIB,
           *[os.path.join(HERE, "csrc", s) for s in SOURCES], "-ldl"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_harness(force="--force" in sys.argv))
