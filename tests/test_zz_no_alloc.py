"""The allocation-free partitioner entry point (agcn_partition_device_noalloc) against the
regular one.

Some hosts cannot let this library allocate device memory: their own allocator owns the whole
GPU, or they cannot take the device-wide stall a cudaMalloc / cudaFree causes, or they forbid
allocation after start-up.  For them the partitioner's tile scratch is a fixed array inside the
library (sized for 2^24 rows).  Because every call on a GPU reuses that one array and it keeps
the previous call's contents, the check is made on consecutive calls with inputs of different
sizes -- a large graph first, then smaller ones whose tiles would see stale values if anything
were read before being rewritten, then a failing call, then a good one again.  Results must be
bit-identical to agcn_partition_device (integer output: no tolerance).

This file is named to be collected last, so that a run that stops at the first failure has
already run every other test.
"""
import ctypes

import numpy as np
import pytest

from conftest import require_cuda

pytestmark = pytest.mark.gpu


def _indptr(rng, n, pool):
    deg = rng.choice(np.asarray(pool), n)
    return np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)


def _partition(lib, fn_name, d_indptr, n_rows, stream):
    import torch
    from accelgcn import _lib
    fn = getattr(lib, fn_name)
    n_blocks = ctypes.c_int64(-1)
    _lib.check(fn(d_indptr.data_ptr(), n_rows, None, 0, ctypes.byref(n_blocks), stream))
    out = torch.full((max(n_blocks.value, 1), 4), -7, dtype=torch.int32, device=d_indptr.device)
    if n_blocks.value:
        _lib.check(fn(d_indptr.data_ptr(), n_rows, out.data_ptr(), n_blocks.value, ctypes.byref(n_blocks), stream))
    torch.cuda.synchronize()
    return out[: n_blocks.value].cpu().numpy()


def test_noalloc_partition_matches_regular_entry_point_on_consecutive_calls():
    import torch
    from accelgcn import _lib
    dev = require_cuda()
    lib = _lib.load()
    stream = torch.cuda.current_stream(dev).cuda_stream
    rng = np.random.default_rng(2024)
    pool = [0, 0, 1, 1, 2, 3, 31, 32, 33, 64, 65, 100, 191, 192, 384, 385, 900, 5000]
    sizes = [1_500_000, 70_000, 2_049, 1, 600_000]           # big first, then smaller, then bigger again
    for call, n in enumerate(sizes):
        ip = _indptr(rng, n, pool if n > 1 else [3])
        if call % 2:
            ip = np.concatenate([[0], np.cumsum(np.sort(np.diff(ip.astype(np.int64))))]).astype(np.int32)
        d_ip = torch.from_numpy(ip).to(dev)
        want = _partition(lib, "agcn_partition_device", d_ip, n, stream)
        got = _partition(lib, "agcn_partition_device_noalloc", d_ip, n, stream)
        assert got.shape == want.shape, (call, n)
        assert np.array_equal(got, want), (call, n)
        # and a second time on the same input, straight after
        again = _partition(lib, "agcn_partition_device_noalloc", d_ip, n, stream)
        assert np.array_equal(again, want), (call, n)


def test_noalloc_partition_errors_then_recovers():
    import torch
    from accelgcn import _lib
    dev = require_cuda()
    lib = _lib.load()
    n_blocks = ctypes.c_int64(0)
    good = torch.from_numpy(np.array([0, 2, 4, 4, 500], dtype=np.int32)).to(dev)
    # beyond the static scratch: rejected with a clear message, before anything is launched
    rc = lib.agcn_partition_device_noalloc(good.data_ptr(), _lib.PARTITION_NOALLOC_MAX_ROWS + 1, None, 0,
                                           ctypes.byref(n_blocks), None)
    assert rc == _lib.ERR_INVALID and b"exceeds" in lib.agcn_last_error()
    # a decreasing indptr sets the error word in the shared scratch ...
    bad = torch.from_numpy(np.array([0, 9, 3, 12], dtype=np.int32)).to(dev)
    assert lib.agcn_partition_device_noalloc(bad.data_ptr(), 3, None, 0, ctypes.byref(n_blocks), None) == _lib.ERR_RANGE
    # ... which the next call must not inherit
    want = _partition(lib, "agcn_partition_device", good, 4, None)
    got = _partition(lib, "agcn_partition_device_noalloc", good, 4, None)
    assert np.array_equal(got, want) and len(got) == 3
    # too small an output buffer reports the needed size, like the regular entry point
    small = torch.zeros((1, 4), dtype=torch.int32, device=dev)
    rc = lib.agcn_partition_device_noalloc(good.data_ptr(), 4, small.data_ptr(), 1, ctypes.byref(n_blocks), None)
    assert rc == _lib.ERR_CAPACITY and n_blocks.value == 3


def test_noalloc_partition_leaves_free_device_memory_unchanged():
    # the property the entry point exists for: after one warm-up call (which may load the kernels),
    # further calls take no device memory -- cudaMemGetInfo reads the same before and after
    import torch
    from accelgcn import _lib
    dev = require_cuda()
    lib = _lib.load()
    rng = np.random.default_rng(7)
    d_ip = torch.from_numpy(_indptr(rng, 300_000, [0, 1, 2, 5, 40, 200, 385, 3000])).to(dev)
    n_blocks = ctypes.c_int64(0)
    _lib.check(lib.agcn_partition_device_noalloc(d_ip.data_ptr(), 300_000, None, 0, ctypes.byref(n_blocks), None))
    out = torch.empty((n_blocks.value, 4), dtype=torch.int32, device=dev)
    _lib.check(lib.agcn_partition_device_noalloc(d_ip.data_ptr(), 300_000, out.data_ptr(), n_blocks.value,
                                                 ctypes.byref(n_blocks), None))          # warm-up, full path
    torch.cuda.synchronize()
    free_before, _total = torch.cuda.mem_get_info(dev)
    for _ in range(3):
        _lib.check(lib.agcn_partition_device_noalloc(d_ip.data_ptr(), 300_000, out.data_ptr(), n_blocks.value,
                                                     ctypes.byref(n_blocks), None))
        assert torch.cuda.mem_get_info(dev)[0] == free_before
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(dev)[0] == free_before
