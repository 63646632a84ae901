"""Two-layer GCN forward  relu(A relu(A X W1) W2)  on the row-sharded operator.

Per layer and per rank:  Z_local = H_local @ W  (agcn_gemm_tf32 on the rows this rank owns),
all-gather Z over the ranks, H'_local = relu(A_shard @ Z)  (the SpMM with its fused ReLU).
The reference stops at the SpMM; the layers are the workload its operator exists for.
"""
from __future__ import annotations

from . import gemm, sharded


class GcnForward:
    def __init__(self, shard: "sharded.ShardedSpmm", weights):
        self.shard = shard
        self.weights = [w.contiguous() for w in weights]
        self._bufs = {}

    def _buf(self, name, rows, cols, like):
        import torch
        b = self._bufs.get(name)
        if b is None or b.shape != (rows, cols):
            b = torch.empty((rows, cols), dtype=torch.float32, device=like.device)
            self._bufs[name] = b
        return b

    def forward(self, x_local, timings=None):
        """x_local: this rank's rows of X [n_local, 128].  Returns this rank's rows of the output."""
        import torch
        sh = self.shard
        h = x_local
        for li, w in enumerate(self.weights):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if timings is not None else None
            if ev: ev[0].record()
            z = gemm.gemm_tf32(h, w, out=self._buf("z", sh.n_local, w.shape[1], h))
            if ev: ev[1].record()
            if sh.world > 1:
                zg = sharded.all_gather_rows(z, sh.cuts, sh.rank, sh.world,
                                             out=self._buf("zg", sh.n_cols, w.shape[1], h), group=sh.group)
            else:
                zg = z
            if ev: ev[2].record()
            h = self._buf(f"h{li % 2}", sh.n_local, w.shape[1], h)
            sh.plan.run(sh.indices, sh.vals, zg, h, dim=w.shape[1], ldx=w.shape[1], ldy=w.shape[1], relu=True)
            if ev:
                ev[3].record()
                timings.append(ev)
        return h
