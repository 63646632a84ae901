"""Degree sort: the Python face of agcn_degree_sort_host/_device.

The reference consumes degree-ordered CSR files (<graph>.new_indptr /
.new_indices, main.cu:62-63) without shipping the code that orders them; this
is that step.  Ascending degree, ties by original row id, optional symmetric
relabel of the column ids.
"""
from __future__ import annotations

import numpy as np

from . import _lib


def degree_sort(indptr, indices, vals=None, relabel_cols: bool = True):
    """Host arrays.  Returns (perm, new_indptr, new_indices, new_vals or None); perm[new_row] = old_row."""
    lib = _lib.load()
    indptr = np.ascontiguousarray(indptr, dtype=np.int32)
    indices = np.ascontiguousarray(indices, dtype=np.int32)
    n_rows, nnz = indptr.shape[0] - 1, indices.shape[0]
    if n_rows <= 0:
        raise IndexError("empty graph")
    v = None if vals is None else np.ascontiguousarray(vals, dtype=np.float32)
    perm = np.empty(n_rows, dtype=np.int32)
    new_indptr = np.empty(n_rows + 1, dtype=np.int32)
    new_indices = np.empty(nnz, dtype=np.int32)
    new_vals = None if v is None else np.empty(nnz, dtype=np.float32)
    _lib.check(lib.agcn_degree_sort_host(
        indptr.ctypes.data, indices.ctypes.data, None if v is None else v.ctypes.data, n_rows, nnz,
        int(bool(relabel_cols)), perm.ctypes.data, new_indptr.ctypes.data, new_indices.ctypes.data,
        None if new_vals is None else new_vals.ctypes.data))
    return perm, new_indptr, new_indices, new_vals


def degree_sort_device(indptr, indices, vals=None, relabel_cols: bool = True, stream=None):
    """torch CUDA tensors (int32 / float32).  Same return convention, on the device."""
    import torch
    lib = _lib.load()
    for t, dt in ((indptr, torch.int32), (indices, torch.int32)) + (((vals, torch.float32),) if vals is not None else ()):
        if not (t.is_cuda and t.dtype == dt and t.is_contiguous()):
            raise TypeError("degree_sort_device needs contiguous CUDA tensors (int32 indptr/indices, float32 vals)")
    dev = indptr.device
    n_rows, nnz = indptr.numel() - 1, indices.numel()
    if n_rows <= 0:
        raise IndexError("empty graph")
    s = stream if stream is not None else torch.cuda.current_stream(dev)
    perm = torch.empty(n_rows, dtype=torch.int32, device=dev)
    new_indptr = torch.empty(n_rows + 1, dtype=torch.int32, device=dev)
    new_indices = torch.empty(nnz, dtype=torch.int32, device=dev)
    new_vals = None if vals is None else torch.empty(nnz, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.agcn_degree_sort_device(
            indptr.data_ptr(), indices.data_ptr(), None if vals is None else vals.data_ptr(), n_rows, nnz,
            int(bool(relabel_cols)), perm.data_ptr(), new_indptr.data_ptr(), new_indices.data_ptr(),
            None if new_vals is None else new_vals.data_ptr(), s.cuda_stream))
    return perm, new_indptr, new_indices, new_vals
