"""Two-layer GCN forward  relu(A relu(A X W1) W2)  on the row blocks of the sharded operator:
the Python face of agcn_gcn2_forward_*.

Per layer and per rank:  Z_block = H_block @ W  (tcgen05 TF32 GEMM on the rows this rank owns),
all-gather of Z (NCCL, slice by slice), H'_block = relu(A_block @ Z) (the SpMM with its fused
ReLU).  The reference stops at the SpMM; the layers are the workload its operator exists for.
Everything is enqueued by the library on the caller's stream; this class owns only the handle.
"""
from __future__ import annotations

import ctypes

from . import _lib, sharded


class GcnForward:
    def __init__(self, shard: "sharded.ShardedSpmm", weights):
        import torch
        if len(weights) != 2:
            raise ValueError("the native forward has two layers")
        self._torch = torch
        self._lib = _lib.load()
        self.shard = shard
        self.weights = [w.contiguous() for w in weights]       # borrowed by the handle: keep alive
        for w in self.weights:
            if tuple(w.shape) != (128, 128) or w.dtype != torch.float32 or not w.is_cuda:
                raise TypeError("weights must be float32 CUDA tensors [128 x 128]")
        h = ctypes.c_void_p()
        with torch.cuda.device(shard.device):
            _lib.check(self._lib.agcn_gcn2_forward_create(ctypes.byref(h), shard._h, self.weights[0].data_ptr(),
                                                          self.weights[1].data_ptr()))
        self._h = h

    def forward(self, x_block, out=None, stream=None):
        """x_block: this rank's block rows of X [rows_per_block, 128].  Returns this rank's block rows of
        the output.  Asynchronous on the current stream; call `status()` after synchronising."""
        torch = self._torch
        if out is None:
            out = torch.empty_like(x_block)
        s = stream if stream is not None else torch.cuda.current_stream(self.shard.device)
        rc = self._lib.agcn_gcn2_forward_run(self._h, x_block.data_ptr(), out.data_ptr(), s.cuda_stream)
        if rc != 0:
            _lib.check(rc)
        return out

    def status(self, timings: bool = False):
        """After a synchronise: raises if a dense transform's bounded wait ran out; with timings=True
        returns per layer (gemm ms, wait for the first exchanged slice ms, spmm ms)."""
        ms = (ctypes.c_float * 6)()
        _lib.check(self._lib.agcn_gcn2_forward_status(self._h, ms if timings else None))
        return [tuple(ms[3 * layer: 3 * layer + 3]) for layer in range(2)] if timings else None

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.agcn_gcn2_forward_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
