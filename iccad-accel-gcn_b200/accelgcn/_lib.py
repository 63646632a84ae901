"""ctypes binding of libaccelgcn.so -- the C ABI declared in include/accelgcn.h.

The library is the product; this module only loads it and declares the
prototypes.  There is no fallback of any kind: if the shared object is missing
or fails to load, importing a function from here raises.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIB = os.path.join(os.path.dirname(_HERE), "lib", "libaccelgcn.so")

OK, ERR_INVALID, ERR_CUDA, ERR_CAPACITY, ERR_RANGE = 0, -1, -2, -3, -4
DEG_BOUND = 384
PARTITION_NOALLOC_MAX_ROWS = 1 << 24

_vp, _i64, _int = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int

# name -> (restype, argtypes); every symbol include/accelgcn.h declares
PROTOTYPES = {
    "agcn_last_error": (ctypes.c_char_p, []),
    "agcn_version": (_int, []),
    "agcn_partition_device": (_int, [_vp, _i64, _vp, _i64, ctypes.POINTER(_i64), _vp]),
    "agcn_partition_host": (_int, [_vp, _i64, _vp, _i64, ctypes.POINTER(_i64)]),
    "agcn_partition_device_noalloc": (_int, [_vp, _i64, _vp, _i64, ctypes.POINTER(_i64), _vp]),
    "agcn_degree_sort_device": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp]),
    "agcn_degree_sort_host": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp]),
    "agcn_spmm_create": (_int, [ctypes.POINTER(_vp), _vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "agcn_spmm_run": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _i64, _int, _vp]),
    "agcn_spmm_run_act": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _i64, _int, _int, _vp]),
    "agcn_spmm_destroy": (_int, [_vp]),
    "agcn_gemm_tf32": (_int, [_vp, _i64, _vp, _vp, _i64, _i64, _int, _int, _vp]),
    "agcn_spmm_plan_info": (_int, [_vp, ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64),
                                  ctypes.POINTER(_int)]),
    "agcn_host_ctx_create": (_int, [ctypes.POINTER(_vp)]),
    "agcn_host_ctx_destroy": (_int, [_vp]),
    "agcn_host_set_graph": (_int, [_vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64]),
    "agcn_host_spmm": (_int, [_vp, _vp, _vp, _int]),
    "agcn_spmm_host": (_int, [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int]),
    "agcn_host_spmm_batch": (_int, [_vp, _int, _vp, _vp, _vp]),
    "agcn_spmm_host_batch": (_int, [_vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp]),
    "agcn_host_last_timing": (_int, [_vp, _vp]),
    "agcn_spmm_tiled_create": (_int, [ctypes.POINTER(_vp), _vp, _vp, _vp, _i64, _i64, _i64, _vp, _int, _vp]),
    "agcn_spmm_tiled_run": (_int, [_vp, _vp, _i64, _vp, _i64, _int, _int, _vp]),
    "agcn_spmm_tiled_run_range": (_int, [_vp, _int, _vp, _i64, _vp, _i64, _int, _int, _vp]),
    "agcn_spmm_tiled_destroy": (_int, [_vp]),
    "agcn_spmm_tiled_info": (_int, [_vp, ctypes.POINTER(_int), ctypes.POINTER(_i64), _vp, ctypes.POINTER(_int)]),
    "agcn_spmm_tiled_suggest": (_int, [_i64, _i64, _i64, _int]),
    "agcn_gemm_tf32_async": (_int, [_vp, _i64, _vp, _vp, _i64, _i64, _int, _int, _vp, _vp]),
    "agcn_gemm_tf32_selftest_timeout": (_int, [_vp, _i64, _vp, _vp, _i64, _i64, _vp]),
    "agcn_gcn_fused_layer": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp]),
    "agcn_balanced_blocks": (_int, [_vp, _i64, _int, _vp, ctypes.POINTER(_i64)]),
    "agcn_dist_unique_id": (_int, [_vp]),
    "agcn_dist_create": (_int, [ctypes.POINTER(_vp), _int, _int, _vp]),
    "agcn_dist_destroy": (_int, [_vp]),
    "agcn_dist_set_graph": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _vp]),
    "agcn_dist_info": (_int, [_vp, ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64),
                             ctypes.POINTER(_i64), ctypes.POINTER(_int), ctypes.POINTER(_int)]),
    "agcn_dist_block_rows": (_int, [_vp, _int, _vp, _vp]),
    "agcn_dist_gather_begin": (_int, [_vp, _int, _vp, _int, _vp]),
    "agcn_dist_spmm_gathered": (_int, [_vp, _int, _vp, _int, _int, _vp]),
    "agcn_dist_spmm_step": (_int, [_vp, _vp, _vp, _int, _int, _vp]),
    "agcn_dist_wait_gathered": (_int, [_vp, _int, _vp]),
    "agcn_dist_spmm_on_gathered": (_int, [_vp, _vp, _vp, _int, _int, _vp]),
    "agcn_dist_gathered": (_int, [_vp, _int, ctypes.POINTER(_vp), ctypes.POINTER(_i64)]),
    "agcn_gcn2_forward_create": (_int, [ctypes.POINTER(_vp), _vp, _vp, _vp]),
    "agcn_gcn2_forward_run": (_int, [_vp, _vp, _vp, _vp]),
    "agcn_gcn2_forward_status": (_int, [_vp, _vp]),
    "agcn_gcn2_forward_destroy": (_int, [_vp]),
    "agcn_probe_gather_bandwidth": (_int, [_i64, _int, _i64, _int, _int, ctypes.POINTER(ctypes.c_double)]),
}
DIST_ID_BYTES = 128
MAX_WORLD = 64

_lib = None


class AccelGcnError(RuntimeError):
    """A call into libaccelgcn.so returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libaccelgcn error {code}: {message}")
        self.code = code


def lib_path() -> str:
    return os.environ.get("ACCELGCN_LIB", DEFAULT_LIB)


def load():
    """Load the shared library (once) and declare every prototype."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} not found: build it with `python iccad-accel-gcn_b200/build.py` "
                "(there is no CPU or PyTorch fallback for this library)")
        lib = ctypes.CDLL(path)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)          # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(code: int) -> None:
    if code != OK:
        raise AccelGcnError(code, load().agcn_last_error().decode("utf-8", "replace"))
