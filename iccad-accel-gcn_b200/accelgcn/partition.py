"""Block-level partitioning: the Python face of agcn_partition_host/_device.

Replaces the per-graph body of the reference's block_level_partition.py
(:38-106).  The result is the same flat int32 array of 4-tuples
(block_degree, block_row_begin, block_loc_begin, block_info), bit for bit.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib


def max_blocks(n_rows: int, nnz: int) -> int:
    """An upper bound on the number of tuples: every row opens at most 1 + degree/384."""
    return int(n_rows) + int(nnz) // _lib.DEG_BOUND


def block_level_partition(indptr) -> np.ndarray:
    """Host arrays in, host array out: int32 [n_blocks, 4].

    `indptr` is the row-pointer array of the degree-ordered CSR (what the
    script reads from <graph>.new_indptr, block_level_partition.py:31)."""
    lib = _lib.load()
    indptr = np.ascontiguousarray(indptr, dtype=np.int32)
    n_rows = indptr.shape[0] - 1
    if n_rows <= 0:
        raise IndexError("empty graph")            # what the reference script raises (:49)
    nnz = int(indptr[-1]) - int(indptr[0])
    cap = max_blocks(n_rows, max(nnz, 0))
    out = np.empty((max(cap, 1), 4), dtype=np.int32)
    n_blocks = ctypes.c_int64(0)
    _lib.check(lib.agcn_partition_host(indptr.ctypes.data, n_rows, out.ctypes.data, cap, ctypes.byref(n_blocks)))
    return out[: n_blocks.value].copy()


def block_level_partition_device(indptr, stream=None):
    """Device tensor in (torch int32 CUDA tensor [n_rows+1]), device tensor out [n_blocks, 4]."""
    import torch
    lib = _lib.load()
    if not (indptr.is_cuda and indptr.dtype == torch.int32 and indptr.is_contiguous()):
        raise TypeError("indptr must be a contiguous int32 CUDA tensor")
    n_rows = indptr.numel() - 1
    if n_rows <= 0:
        raise IndexError("empty graph")
    s = stream if stream is not None else torch.cuda.current_stream(indptr.device)
    n_blocks = ctypes.c_int64(0)
    with torch.cuda.device(indptr.device):
        _lib.check(lib.agcn_partition_device(indptr.data_ptr(), n_rows, None, 0, ctypes.byref(n_blocks), s.cuda_stream))
        out = torch.empty((n_blocks.value, 4), dtype=torch.int32, device=indptr.device)
        if n_blocks.value:
            _lib.check(lib.agcn_partition_device(indptr.data_ptr(), n_rows, out.data_ptr(), n_blocks.value,
                                                 ctypes.byref(n_blocks), s.cuda_stream))
    return out
