import hashlib
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "iccad-accel-gcn_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")

# fp32 tolerance of the SpMM parity gate: rel 1e-4 / abs 1e-5
RTOL, ATOL = 1e-4, 1e-5


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


def pytest_collection_modifyitems(config, items):
    # files whose name starts with test_zz_ are collected last on purpose
    items.sort(key=lambda it: os.path.basename(str(it.fspath)).startswith("test_zz_"))


@pytest.fixture(scope="session", autouse=True)
def built_library():
    """libaccelgcn.so is compiled from csrc/ when it is missing or older than its sources (nvcc
    cross-compiles without a GPU).  Nothing falls back to anything else if that fails."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("agcn_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


@pytest.fixture(scope="session")
def kat():
    """Degree sequences and hashes of the 16 golden .block4 files of the reference."""
    with open(os.path.join(GOLDEN, "block4_kat.json")) as fh:
        return json.load(fh)


@pytest.fixture(scope="session")
def edge_cases():
    """Edge-case indptr arrays with the outputs of the unmodified reference script."""
    z = np.load(os.path.join(GOLDEN, "partition_edge_cases.npz"))
    names = sorted(k[len("indptr__"):] for k in z.files if k.startswith("indptr__"))
    return {n: (z["indptr__" + n], z["block4__" + n].reshape(-1, 4)) for n in names}


def kat_indptr(entry) -> np.ndarray:
    deg = np.concatenate([np.zeros(entry["leading_zero_rows"], dtype=np.int64),
                          np.repeat(np.asarray(entry["degrees"], dtype=np.int64),
                                    np.asarray(entry["counts"], dtype=np.int64))])
    return np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)


def sha256_block4(block4) -> str:
    return hashlib.sha256(np.ascontiguousarray(block4, dtype=np.int32).tobytes()).hexdigest()


def spmm_close(y, ref, scale=None):
    """|y - ref| <= ATOL * max(1, scale) + RTOL * |ref|, elementwise.

    `scale` (per row, optional) is sum_j |a_ij| * max|x|: fp32 accumulation error grows with
    it, so for rows whose absolute sum exceeds 1 the absolute term is scaled by it -- the
    reference's own fp32 kernel has the same property."""
    y, ref = np.asarray(y, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    atol = ATOL if scale is None else ATOL * np.maximum(1.0, np.asarray(scale, dtype=np.float64))[:, None]
    return np.abs(y - ref) <= atol + RTOL * np.abs(ref)


def row_abs_scale(indptr, val, x):
    indptr = np.asarray(indptr, dtype=np.int64)
    s = np.add.reduceat(np.concatenate([np.abs(val).astype(np.float64), [0.0]]),
                        np.minimum(indptr[:-1], len(val)))
    s[np.diff(indptr) == 0] = 0.0
    return s * float(np.abs(x).max())


def require_cuda():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device (there is no CPU fallback to test)"
    return torch.device("cuda:0")
