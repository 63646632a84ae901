"""Two-layer GCN forward  relu(A relu(A X W1) W2)  on the row-sharded operator.

Per layer and per rank:  Z_local = H_local @ W  (agcn_gemm_tf32 on the rows this rank owns),
all-gather Z over the ranks, H'_local = relu(A_shard @ Z)  (the SpMM with its fused ReLU).
The reference stops at the SpMM; the layers are the workload its operator exists for.
"""
from __future__ import annotations

from . import gemm, sharded


class GcnForward:
    """panel_cols: with more than one rank the all-gather of X*W is the longest part of a layer and
    the SpMM cannot start on a row before all of its columns' rows have arrived -- but it can start
    on a COLUMN panel as soon as that panel has.  With panel_cols = 32 or 64, X*W is exchanged in
    panels of that many columns and the SpMM of panel p runs while panel p+1 is still in flight.
    Off by default (panel_cols=None: exchange and multiply all columns at once): measured on two
    B200s at N = 5e6 the panelled schedule was slower (10.5 against 8.4 ms per layer) -- four
    32-column passes over an operand far larger than L2 cost more than one 128-column pass, and
    they compete with the collective for HBM bandwidth while it runs."""

    def __init__(self, shard: "sharded.ShardedSpmm", weights, panel_cols=None):
        self.shard = shard
        self.weights = [w.contiguous() for w in weights]
        self.panel_cols = panel_cols
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
            width = w.shape[1]
            h_next = self._buf(f"h{li % 2}", sh.n_local, width, h)
            if self.panel_cols is None:
                if sh.world > 1:
                    zg = sharded.all_gather_rows(z, sh.cuts, sh.rank, sh.world,
                                                 out=self._buf("zg", sh.n_cols, width, h), group=sh.group)
                else:
                    zg = z
                if ev: ev[2].record()
                sh.plan.run(sh.indices, sh.vals, zg, h_next, dim=width, ldx=width, ldy=width, relu=True)
            else:
                pc = self.panel_cols
                pending = []
                for c0 in range(0, width, pc):
                    c1 = min(width, c0 + pc)
                    zp = self._buf(f"zp{c0}", sh.n_local, c1 - c0, h)
                    zp.copy_(z[:, c0:c1])
                    if sh.world > 1:
                        pending.append(sharded.all_gather_rows(zp, sh.cuts, sh.rank, sh.world,
                                                               out=self._buf(f"zg{c0}", sh.n_cols, c1 - c0, h),
                                                               group=sh.group, async_op=True))
                    else:
                        pending.append((zp, None))
                if ev: ev[2].record()          # all exchanges started; their time shows up in the SpMM span
                for (zg, work), c0 in zip(pending, range(0, width, pc)):
                    c1 = min(width, c0 + pc)
                    if work is not None:
                        work.wait()
                    sh.plan.run(sh.indices, sh.vals, zg, h_next[:, c0:c1], dim=c1 - c0, ldx=c1 - c0, ldy=width, relu=True)
            h = h_next
            if ev:
                ev[3].record()
                timings.append(ev)
        return h
