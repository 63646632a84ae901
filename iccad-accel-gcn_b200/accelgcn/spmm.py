"""SpMM plug-in: the Python face of agcn_spmm_create / _run / _destroy.

`SpmmAccel` mirrors the reference's SPMM_ACCEL class (spmm_accel.h:4-20 over
spmm_base.h:6-65): the constructor borrows the caller's arrays,
`do_test(timing, dim)` prepares the .block4 metadata and runs or times the
kernel with the reference's protocol (4 warm-up + 4 timed launches, mean
seconds; spmm_base.h:34-63), `run(dim)` is one asynchronous launch.
"""
from __future__ import annotations

import ctypes
import os
import time

import numpy as np

from . import _lib, graphio


class SpmmPlan:
    """Owner of an agcn_spmm_plan handle (validated .block4 + launch plan)."""

    def __init__(self, block4, indices, n_rows: int, n_cols: int, stream=None):
        import torch
        lib = _lib.load()
        if not (block4.is_cuda and block4.dtype == torch.int32 and block4.is_contiguous()):
            raise TypeError("block4 must be a contiguous int32 CUDA tensor")
        self._lib = lib
        self.block4 = block4            # keep alive: the plan borrows it
        self.device = block4.device
        self._dev_index = block4.device.index if block4.device.index is not None else torch.cuda.current_device()
        self.n_rows, self.n_cols = int(n_rows), int(n_cols)
        self.n_blocks = block4.numel() // 4
        self.nnz = int(indices.numel())
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(lib.agcn_spmm_create(ctypes.byref(h), block4.data_ptr(), self.n_blocks, indices.data_ptr(),
                                            self.n_rows, self.n_cols, self.nnz, s.cuda_stream))
        self._h = h

    def run(self, indices, vals, x, y, dim: int | None = None, ldx: int | None = None, ldy: int | None = None,
            stream=None, relu: bool = False) -> None:
        import torch
        dim = int(x.shape[1] if dim is None else dim)
        ldx = int(x.stride(0) if ldx is None and x.dim() == 2 else (dim if ldx is None else ldx))
        ldy = int(y.stride(0) if ldy is None and y.dim() == 2 else (dim if ldy is None else ldy))
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        args = (self._h, indices.data_ptr(), vals.data_ptr(), x.data_ptr(), ldx, y.data_ptr(), ldy, dim,
                1 if relu else 0, s.cuda_stream)
        if torch.cuda.current_device() == self._dev_index:      # the usual case: no device switch needed
            rc = self._lib.agcn_spmm_run_act(*args)
        else:
            with torch.cuda.device(self.device):
                rc = self._lib.agcn_spmm_run_act(*args)
        if rc != 0:
            _lib.check(rc)

    def info(self) -> dict:
        a, b, c, d = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int()
        _lib.check(self._lib.agcn_spmm_plan_info(self._h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), ctypes.byref(d)))
        return {"n_units": a.value, "n_carry": b.value, "n_zero_rows": c.value, "launches_last_run": d.value}

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.agcn_spmm_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class TiledSpmmPlan:
    """Column-tiled product (agcn_spmm_tiled_*): A regrouped by column range so that every launch
    gathers from one L2-resident slab of X; the first range stores Y, later ranges add to it.
    `bounds` are the ascending column ids that start each range (from 0 to n_cols); without them
    the library's suggestion for `dim` columns is used (equal ranges)."""

    def __init__(self, indptr, indices, vals, n_rows: int, n_cols: int, bounds=None, dim: int = 128, stream=None):
        import torch
        lib = _lib.load()
        self._lib, self.device = lib, indptr.device
        nnz = int(indices.numel())
        if bounds is None:
            k = lib.agcn_spmm_tiled_suggest(int(n_rows), int(n_cols), nnz, int(dim))
            bounds = [int(n_cols) * i // k for i in range(k + 1)]
        self.bounds = np.ascontiguousarray(bounds, dtype=np.int32)
        self.n_rows, self.n_cols = int(n_rows), int(n_cols)
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(lib.agcn_spmm_tiled_create(ctypes.byref(h), indptr.data_ptr(), indices.data_ptr(), vals.data_ptr(),
                                                  self.n_rows, self.n_cols, nnz, self.bounds.ctypes.data,
                                                  len(self.bounds) - 1, s.cuda_stream))
        self._h = h

    def run(self, x, y, relu: bool = False, stream=None, only_range: int | None = None) -> None:
        import torch
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        dim, ldx, ldy = int(x.shape[1]), int(x.stride(0)), int(y.stride(0))
        with torch.cuda.device(self.device):
            if only_range is None:
                rc = self._lib.agcn_spmm_tiled_run(self._h, x.data_ptr(), ldx, y.data_ptr(), ldy, dim, 1 if relu else 0, s.cuda_stream)
            else:
                rc = self._lib.agcn_spmm_tiled_run_range(self._h, int(only_range), x.data_ptr(), ldx, y.data_ptr(), ldy, dim,
                                                         1 if relu else 0, s.cuda_stream)
        if rc != 0:
            _lib.check(rc)

    def info(self) -> dict:
        k, nb, ln = ctypes.c_int(), ctypes.c_int64(), ctypes.c_int()
        rn = (ctypes.c_int64 * 32)()
        _lib.check(self._lib.agcn_spmm_tiled_info(self._h, ctypes.byref(k), ctypes.byref(nb), rn, ctypes.byref(ln)))
        return {"n_ranges": k.value, "n_blocks": nb.value, "range_nnz": list(rn)[: k.value], "launches_last_run": ln.value}

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.agcn_spmm_tiled_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def spmm(block4, indices, vals, x, n_rows: int | None = None, out=None):
    """Y = A @ X on the device.  block4 [n_blocks,4] int32, indices int32, vals fp32, x [n_cols, dim] fp32."""
    import torch
    n_rows = int(x.shape[0] if n_rows is None else n_rows)
    y = out if out is not None else torch.empty((n_rows, x.shape[1]), dtype=torch.float32, device=x.device)
    plan = SpmmPlan(block4, indices, n_rows, x.shape[0])
    try:
        plan.run(indices, vals, x, y)
    finally:
        torch.cuda.current_stream(x.device).synchronize()
        plan.close()
    return y


class SpmmAccel:
    """Drop-in mirror of SPMM_ACCEL.

    Constructor arguments follow SPMM_BASE (spmm_base.h:9): graph name, row
    pointers, column ids, values, dense input, dense output, vertex count, edge
    count, buffer capacity in columns.  The arrays are borrowed CUDA tensors;
    vin / vout are re-read as [num_v x dim] row-major for whatever dim each call
    names (main.cu:84-88,137).  `meta_dir` is where <graph>.block4 lives
    (the reference hard-codes ../block_level_meta/, spmm_accel.cu:122)."""

    TIMES = 4   # spmm_base.h:44

    def __init__(self, graph, ptr, idx, val, vin, vout, num_v, num_e, dim, meta_dir="../block_level_meta/"):
        self._graph, self.ptr, self.idx, self.val = graph, ptr, idx, val
        self.vin, self.vout = vin, vout
        self.num_v, self.num_e, self.dim = int(num_v), int(num_e), int(dim)
        self.meta_dir = meta_dir
        self._plan = None

    # -- SPMM_ACCEL::run (spmm_accel.cu:104-108): one asynchronous launch, no sync
    def run(self, dim: int) -> None:
        self._plan.run(self.idx, self.val, self.vin, self.vout, dim=dim, ldx=dim, ldy=dim)

    # -- SPMM_BASE::timing_body (spmm_base.h:34-63)
    def _timing_body(self, timing: bool, dim: int) -> float:
        import torch
        if not timing:
            self.run(dim)
            torch.cuda.synchronize(self.vin.device)
            return 0.0
        for _ in range(self.TIMES):
            self.run(dim)
        torch.cuda.synchronize(self.vin.device)
        total = 0.0
        for _ in range(self.TIMES):
            t0 = time.perf_counter()
            self.run(dim)
            torch.cuda.synchronize(self.vin.device)
            total += time.perf_counter() - t0
        return total / self.TIMES

    # -- SPMM_ACCEL::do_test (spmm_accel.cu:110-139)
    def do_test(self, timing: bool, dim: int) -> float:
        import torch
        path = os.path.join(self.meta_dir, self._graph + ".block4")
        block4 = torch.from_numpy(np.ascontiguousarray(graphio.read_block4(path))).to(self.vin.device)
        self._plan = SpmmPlan(block4, self.idx, self.num_v, self.num_v)
        try:
            return self._timing_body(timing, dim)
        finally:
            self._plan.close()
            self._plan = None


class HostSpmm:
    """Host-buffer call (agcn_spmm_host): numpy arrays in, numpy array out, every
    byte crossing PCIe inside the call.  Keeps its device buffers between calls."""

    def __init__(self):
        self._lib = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(self._lib.agcn_host_ctx_create(ctypes.byref(h)))
        self._h = h

    def set_graph(self, block4, indices, vals, n_rows: int, n_cols: int) -> None:
        """Upload .block4, column ids and values and build the plan (the constructor's share of the plug-in)."""
        self._n_rows, self._n_cols = int(n_rows), int(n_cols)
        _lib.check(self._lib.agcn_host_set_graph(self._h, _addr(block4), _numel(block4) // 4, _addr(indices),
                                                 _addr(vals), n_rows, n_cols, _numel(indices)))

    def run(self, x, out=None):
        """One product on host operands: X up, SpMM, Y down."""
        dim = x.shape[1]
        if x.shape[0] != self._n_cols:
            raise ValueError("X has the wrong number of rows")
        y = out if out is not None else np.empty((self._n_rows, dim), dtype=np.float32)
        _lib.check(self._lib.agcn_host_spmm(self._h, _addr(x), _addr(y), dim))
        return y

    def run_batch(self, xs, outs=None):
        """Several products enqueued together (agcn_host_spmm_batch): uploads, kernels and downloads overlap."""
        n = len(xs)
        for x in xs:
            if x.shape[0] != self._n_cols:
                raise ValueError("X has the wrong number of rows")
        ys = outs if outs is not None else [np.empty((self._n_rows, x.shape[1]), dtype=np.float32) for x in xs]
        px = (ctypes.c_void_p * n)(*[_addr(x) for x in xs])
        py = (ctypes.c_void_p * n)(*[_addr(y) for y in ys])
        dims = (ctypes.c_int * n)(*[int(x.shape[1]) for x in xs])
        _lib.check(self._lib.agcn_host_spmm_batch(self._h, n, px, py, dims))
        return ys

    def step_batch(self, block4, indices, vals, xs, n_rows: int, outs=None):
        """The graph and several products in one call (agcn_spmm_host_batch): A goes up in ranges and
        every range is multiplied as soon as it has arrived."""
        n = len(xs)
        n_cols = xs[0].shape[0]
        self._n_rows, self._n_cols = int(n_rows), int(n_cols)
        ys = outs if outs is not None else [np.empty((n_rows, x.shape[1]), dtype=np.float32) for x in xs]
        px = (ctypes.c_void_p * n)(*[_addr(x) for x in xs])
        py = (ctypes.c_void_p * n)(*[_addr(y) for y in ys])
        dims = (ctypes.c_int * n)(*[int(x.shape[1]) for x in xs])
        _lib.check(self._lib.agcn_spmm_host_batch(self._h, _addr(block4), _numel(block4) // 4, _addr(indices), _addr(vals),
                                                  n_rows, n_cols, _numel(indices), n, px, py, dims))
        return ys

    def last_timing(self) -> dict:
        """Milliseconds of the last streamed step_batch call, from the start of its uploads (agcn_host_last_timing)."""
        ms = (ctypes.c_float * 6)()
        _lib.check(self._lib.agcn_host_last_timing(self._h, ms))
        keys = ("a_uploaded", "first_kernel_started", "last_kernel_finished", "last_y_downloaded", "host_plan_built", "host_all_enqueued")
        return dict(zip(keys, (float(v) for v in ms)))

    def __call__(self, block4, indices, vals, x, n_rows: int, out=None):
        n_cols, dim = x.shape
        y = out if out is not None else np.empty((n_rows, dim), dtype=np.float32)
        _lib.check(self._lib.agcn_spmm_host(self._h, _addr(block4), _numel(block4) // 4, _addr(indices), _addr(vals),
                                            _addr(x), _addr(y), n_rows, n_cols, _numel(indices), dim))
        return y

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.agcn_host_ctx_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _addr(a) -> int:
    """Address of a host array: numpy array or (pinned) CPU torch tensor."""
    if isinstance(a, np.ndarray):
        if not a.flags["C_CONTIGUOUS"]:
            raise TypeError("array must be C-contiguous")
        return a.ctypes.data
    if a.is_cuda or not a.is_contiguous():
        raise TypeError("host call needs contiguous CPU tensors")
    return a.data_ptr()


def _numel(a) -> int:
    return int(a.size) if isinstance(a, np.ndarray) else int(a.numel())
