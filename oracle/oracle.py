"""TEST INFRASTRUCTURE ONLY: CPU oracle for the Accel-GCN hot path.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
import this module -- as the checker or as a reported baseline, never as the
thing shipped or measured.  The product library never falls back to it.

What is restated, and from where in the reference:

* ``partition_py``   -- block_level_partition.py:7-21,48-103 in pure Python
  (small inputs only; it is as slow as the script it restates).
* ``partition``      -- the same walk in C (oracle/partition_oracle.c).
* ``degree_sort``    -- the degree ordering the reference *assumes* but does
  not ship (its inputs are the pre-sorted ``.new_indptr/.new_indices`` files,
  main.cu:62-63).  PARITY UNPINNED for this one function: the only fact the
  reference pins is ascending degree order (every golden ``.block4`` is
  non-decreasing in degree); the tie-break (stable, by original row id) and
  the symmetric column relabel are this project's choice.
* ``spmm_block4``    -- spmm_accel.cu:16-102 thread for thread, fp32.
* ``spmm_csr``       -- CSR x dense with fp64 accumulation (the arithmetic of
  the harness check against cusparseSpMM, main.cu:141-156).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

# Where the reference source tree (an ICCAD-Accel-GCN checkout) lies, when it is needed: building
# oracle/_ref, regenerating fixtures, the live-script tests.  Set ACCELGCN_REFERENCE to name it; when
# the variable is unset a checkout placed beside this repository (../reference) is used if it exists.
# Nothing that runs on a GPU box needs it, and everything that does skips cleanly when it is None.
def _find_reference():
    named = os.environ.get("ACCELGCN_REFERENCE")
    if named:
        return named if os.path.isfile(os.path.join(named, "block_level_partition.py")) else None
    beside = os.path.normpath(os.path.join(_HERE, os.pardir, os.pardir, "reference"))
    return beside if os.path.isfile(os.path.join(beside, "block_level_partition.py")) else None


REFERENCE_DIR = _find_reference()

DEG_BOUND = 12 * 32   # block_level_partition.py:7
NUM_WARPS = 12        # block_level_partition.py:8


def build(force: bool = False) -> str:
    """Compile oracle/liboracle.so with gcc (no GPU needed)."""
    so = os.path.join(_HERE, "liboracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("partition_oracle.c", "spmm_oracle.c")]
    if force or not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return so


def _lib():
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(build())
        i32p, f32p, i64 = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_float), ctypes.c_int64
        lib.agcn_oracle_partition.restype = i64
        lib.agcn_oracle_partition.argtypes = [i32p, i64, i32p, i64]
        lib.agcn_oracle_pattern.restype = ctypes.c_int
        lib.agcn_oracle_pattern.argtypes = [i32p, i32p]
        lib.agcn_oracle_spmm_block4.restype = ctypes.c_int
        lib.agcn_oracle_spmm_block4.argtypes = [i32p, i64, i32p, f32p, f32p, f32p, i64, i64, i64, ctypes.c_int]
        for name in ("agcn_oracle_spmm_csr_f64acc", "agcn_oracle_spmm_csr_f32"):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [i32p, i32p, f32p, f32p, f32p, i64, i64, ctypes.c_int]
        lib.agcn_oracle_num_threads.restype = ctypes.c_int
        _LIB = lib
    return _LIB


def _p(a, ct):
    return a.ctypes.data_as(ctypes.POINTER(ct))


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def pattern_tables():
    """(warp_nz, block_rows) lists of length 192 -- block_level_partition.py:7-21."""
    warp_nz, block_rows = [0], [0]
    warp_max_nz = DEG_BOUND // NUM_WARPS
    factor = (1, 2, 3, 4, 6, 12)
    jf, i = 0, 1
    while i < DEG_BOUND // 2:
        if factor[jf] * warp_max_nz >= i:
            warp_nz.append((i + factor[jf] - 1) // factor[jf])
            block_rows.append(NUM_WARPS // factor[jf])
            i += 1
        else:
            jf += 1
    return warp_nz, block_rows


def partition_py(indptr) -> np.ndarray:
    """Pure-Python restatement of the walk at block_level_partition.py:48-103.

    Returns an int32 array of shape (n_blocks, 4): degree, row_begin,
    loc_begin, info.  Raises IndexError on an empty graph as the script does."""
    indptr = np.asarray(indptr, dtype=np.int64)
    deg = np.diff(indptr)
    n = len(deg)
    warp_nz, block_rows = pattern_tables()
    out = []
    cur_row, cur_loc = 0, 0
    if n == 0:
        raise IndexError("empty graph")
    while True:
        d = int(deg[cur_row])
        if d == 0:
            cur_row += 1
        elif 1 <= d <= DEG_BOUND:
            w_nz = DEG_BOUND // NUM_WARPS if d >= len(warp_nz) else warp_nz[d]
            b_row = 1 if d >= len(block_rows) else block_rows[d]
            row_begin, loc_begin, j = cur_row, cur_loc, 0
            while deg[cur_row] == d:
                cur_row += 1
                j += 1
                if j == b_row or cur_row == n:
                    break
            cur_loc += j * d
            out.append((d, row_begin, loc_begin, (w_nz << 16) + j))
        elif d > DEG_BOUND:
            done = 0
            while done < d:
                take = min(DEG_BOUND, d - done)
                out.append((d, cur_row, cur_loc, take))
                cur_loc += take
                done += take
            cur_row += 1
        else:
            raise ValueError("negative degree")
        if cur_row == n:
            break
    return np.asarray(out, dtype=np.int64).reshape(-1, 4).astype(np.int32)


def partition(indptr) -> np.ndarray:
    """C restatement of the same walk (oracle/partition_oracle.c)."""
    indptr = _i32(indptr)
    n = len(indptr) - 1
    lib = _lib()
    cnt = lib.agcn_oracle_partition(_p(indptr, ctypes.c_int32), n, None, 0)
    if cnt < 0:
        raise ValueError(f"oracle partition failed ({cnt})")
    out = np.empty((cnt, 4), dtype=np.int32)
    lib.agcn_oracle_partition(_p(indptr, ctypes.c_int32), n, _p(out, ctypes.c_int32), cnt)
    return out


def degree_sort(indptr, indices, vals=None, relabel_cols=True):
    """Stable ascending sort of the rows by degree, with optional symmetric
    relabel of the column ids (new id of old row r = its position in the
    sorted order).  Returns (perm, new_indptr, new_indices, new_vals) where
    perm[new_row] = old_row.  Columns keep their within-row order."""
    indptr = np.asarray(indptr, dtype=np.int64)
    indices = np.asarray(indices)
    deg = np.diff(indptr)
    perm = np.argsort(deg, kind="stable")
    new_deg = deg[perm]
    new_indptr = np.zeros(len(deg) + 1, dtype=np.int64)
    np.cumsum(new_deg, out=new_indptr[1:])
    # gather every row's slice: position p of the output belongs to new row r
    row_of = np.repeat(np.arange(len(deg)), new_deg)
    src = indptr[perm][row_of] + (np.arange(new_indptr[-1]) - new_indptr[row_of])
    new_indices = indices[src]
    if relabel_cols:
        inv = np.empty(len(deg), dtype=np.int64)
        inv[perm] = np.arange(len(deg))
        new_indices = inv[new_indices]
    new_vals = None if vals is None else np.asarray(vals)[src]
    return (perm.astype(np.int32), new_indptr.astype(np.int32),
            new_indices.astype(np.int32), new_vals)


def spmm_block4(block4, idx, val, x, n_rows, y0=None) -> np.ndarray:
    """The reference kernel, thread for thread, on the CPU (fp32)."""
    block4, idx, val, x = _i32(block4).reshape(-1, 4), _i32(idx), _f32(val), _f32(x)
    dim = x.shape[1]
    y = np.zeros((n_rows, dim), dtype=np.float32) if y0 is None else _f32(y0).copy()
    rc = _lib().agcn_oracle_spmm_block4(_p(block4, ctypes.c_int32), len(block4), _p(idx, ctypes.c_int32),
                                        _p(val, ctypes.c_float), _p(x, ctypes.c_float), _p(y, ctypes.c_float),
                                        n_rows, x.shape[0], len(idx), dim)
    if rc != 0:
        raise ValueError("oracle spmm_block4: index out of range")
    return y


def spmm_csr(indptr, idx, val, x, f32_accumulate=False) -> np.ndarray:
    """CSR x dense; fp64 accumulation unless f32_accumulate (the timed baseline)."""
    indptr, idx, val, x = _i32(indptr), _i32(idx), _f32(val), _f32(x)
    n, dim = len(indptr) - 1, x.shape[1]
    y = np.empty((n, dim), dtype=np.float32)
    fn = _lib().agcn_oracle_spmm_csr_f32 if f32_accumulate else _lib().agcn_oracle_spmm_csr_f64acc
    rc = fn(_p(indptr, ctypes.c_int32), _p(idx, ctypes.c_int32), _p(val, ctypes.c_float),
            _p(x, ctypes.c_float), _p(y, ctypes.c_float), n, x.shape[0], dim)
    if rc != 0:
        raise ValueError("oracle spmm_csr: column index out of range")
    return y


def num_threads() -> int:
    return int(_lib().agcn_oracle_num_threads())


def use_all_host_threads() -> int:
    """Let the OpenMP loops use every core this process may run on, whatever OMP_NUM_THREADS says."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    _lib().agcn_oracle_set_num_threads(n)
    return num_threads()


# --------------------------------------------------------------------------
# The reference's own CUDA kernels, compiled from its sources into
# oracle/_ref/libref_accel.so by `make -C oracle ref` (needs the reference
# tree at build time only).  Used on a GPU box as the parity oracle for the
# SpMM and as the kernel to beat.
# --------------------------------------------------------------------------
_REF = None


def ref_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libref_accel.so"))


def _ref():
    global _REF
    if _REF is None:
        lib = ctypes.CDLL(os.path.join(_HERE, "_ref", "libref_accel.so"))
        i32p, f32p, i64 = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_float), ctypes.c_int64
        dp = ctypes.POINTER(ctypes.c_double)
        lib.ref_accel_spmm.restype = ctypes.c_int
        lib.ref_accel_spmm.argtypes = [ctypes.c_char_p, i32p, i64, i32p, i32p, f32p, f32p, f32p, i64, i64,
                                       ctypes.c_int, ctypes.c_int, dp]
        lib.ref_cusparse_spmm.restype = ctypes.c_int
        lib.ref_cusparse_spmm.argtypes = [i32p, i32p, f32p, f32p, f32p, i64, i64, ctypes.c_int, ctypes.c_int, dp]
        lib.ref_gnna_time.restype = ctypes.c_int
        lib.ref_gnna_time.argtypes = [ctypes.c_char_p, i32p, i32p, f32p, f32p, i64, i64, ctypes.c_int, dp]
        _REF = lib
    return _REF


def ref_accel_spmm(block4, indptr, idx, val, x, timing=False, workdir=None):
    """Reference spmm_kernel_accel on a zeroed Y.  Returns Y (timing=False) or mean seconds per launch."""
    import tempfile
    block4, indptr, idx, val, x = _i32(block4).reshape(-1, 4), _i32(indptr), _i32(idx), _f32(val), _f32(x)
    n, dim = len(indptr) - 1, x.shape[1]
    y = np.zeros((n, dim), dtype=np.float32)
    sec = ctypes.c_double(0.0)
    with tempfile.TemporaryDirectory() as tmp:
        rc = _ref().ref_accel_spmm((workdir or tmp).encode(), _p(block4, ctypes.c_int32), len(block4),
                                   _p(indptr, ctypes.c_int32), _p(idx, ctypes.c_int32), _p(val, ctypes.c_float),
                                   _p(x, ctypes.c_float), _p(y, ctypes.c_float), n, len(idx), dim, int(timing),
                                   ctypes.byref(sec))
    if rc != 0:
        raise RuntimeError(f"ref_accel_spmm failed ({rc})")
    return sec.value if timing else y


def ref_cusparse_spmm(indptr, idx, val, x, timing=False):
    indptr, idx, val, x = _i32(indptr), _i32(idx), _f32(val), _f32(x)
    n, dim = len(indptr) - 1, x.shape[1]
    y = np.zeros((n, dim), dtype=np.float32)
    sec = ctypes.c_double(0.0)
    rc = _ref().ref_cusparse_spmm(_p(indptr, ctypes.c_int32), _p(idx, ctypes.c_int32), _p(val, ctypes.c_float),
                                  _p(x, ctypes.c_float), _p(y, ctypes.c_float), n, len(idx), dim, int(timing),
                                  ctypes.byref(sec))
    if rc != 0:
        raise RuntimeError(f"ref_cusparse_spmm failed ({rc})")
    return sec.value if timing else y


def ref_gnna_time(indptr, idx, val, x):
    import tempfile
    indptr, idx, val, x = _i32(indptr), _i32(idx), _f32(val), _f32(x)
    n, dim = len(indptr) - 1, x.shape[1]
    sec = ctypes.c_double(0.0)
    with tempfile.TemporaryDirectory() as tmp:
        rc = _ref().ref_gnna_time(tmp.encode(), _p(indptr, ctypes.c_int32), _p(idx, ctypes.c_int32),
                                  _p(val, ctypes.c_float), _p(x, ctypes.c_float), n, len(idx), dim, ctypes.byref(sec))
    if rc != 0:
        raise RuntimeError(f"ref_gnna_time failed ({rc})")
    return sec.value
