"""1D row-sharded multi-GPU SpMM: one process per GPU, torch.distributed for the
exchange, libaccelgcn.so for every kernel.

The degree-ordered matrix A is cut at row boundaries into one contiguous row
range per rank, balanced by nonzeros (not rows).  Each rank keeps its rows of
A, its own `.block4` metadata (the partitioner run on the shard's row
pointers -- the format is unchanged, row and nonzero offsets are shard-local)
and the same rows of the dense operand.  One step is: all-gather the dense
operand (the only exchange the path has), then the local SpMM.

Balancing by nonzeros makes the row counts very uneven (the first rank owns
most of the light rows), so the exchange is an all-gather with a different
block size per rank, straight into the [n x dim] operand in global row order:
nothing is padded and column ids keep their global numbering.

The reference has no multi-GPU code; this follows its single-GPU operator
(spmm_accel.cu) shard by shard.
"""
from __future__ import annotations

import numpy as np


def nnz_balanced_cuts(indptr, n_parts: int) -> np.ndarray:
    """Row cut points c[0]=0 <= ... <= c[n_parts]=n_rows such that every range
    [c[k], c[k+1]) holds about nnz / n_parts nonzeros.  Cuts fall on row
    boundaries (a row is never split); indptr is a host array."""
    indptr = np.asarray(indptr, dtype=np.int64)
    n_rows = len(indptr) - 1
    nnz = int(indptr[-1] - indptr[0])
    targets = indptr[0] + (np.arange(1, n_parts, dtype=np.int64) * nnz) // n_parts
    inner = np.searchsorted(indptr, targets, side="left")
    cuts = np.concatenate([[0], np.clip(inner, 0, n_rows), [n_rows]]).astype(np.int64)
    return np.maximum.accumulate(cuts)


def shard_rows(indptr, indices, vals, cuts, rank: int):
    """The rows [cuts[rank], cuts[rank+1]) of a CSR matrix, row pointers rebased to 0."""
    r0, r1 = int(cuts[rank]), int(cuts[rank + 1])
    p0, p1 = int(indptr[r0]), int(indptr[r1])
    return indptr[r0:r1 + 1] - indptr[r0], indices[p0:p1], vals[p0:p1]


def all_gather_rows(x_local, cuts, rank: int, world_size: int, out=None, group=None, async_op: bool = False):
    """All-gather row blocks of different heights: rank r contributes rows [cuts[r], cuts[r+1]) of
    the [n x dim] result.  On NCCL this is one all-gather call with per-rank sizes (grouped
    broadcasts inside the library); on other backends (the gloo CPU tests) one broadcast per rank."""
    import torch
    import torch.distributed as dist
    n, dim = int(cuts[-1]), x_local.shape[1]
    if out is None:
        out = torch.empty((n, dim), dtype=x_local.dtype, device=x_local.device)
    if world_size == 1:
        out.copy_(x_local)
        return out
    blocks = [out[int(cuts[r]):int(cuts[r + 1])] for r in range(world_size)]
    if dist.get_backend(group) == "nccl":
        work = dist.all_gather(blocks, x_local.contiguous(), group=group, async_op=async_op)
        return (out, work) if async_op else out
    else:
        blocks[rank].copy_(x_local)
        for r in range(world_size):
            if blocks[r].numel():
                dist.broadcast(blocks[r], src=dist.get_global_rank(group, r) if group is not None else r, group=group)
    return (out, None) if async_op else out


def even_rows(n: int, world_size: int) -> int:
    """Rows per rank when the dense operand is block-distributed evenly (the last block is padded)."""
    return -(-int(n) // int(world_size))


def all_gather_even(x_block, world_size: int, out=None, group=None, async_op: bool = False):
    """All-gather of equal blocks [rows_per_rank x dim] into [world_size * rows_per_rank x dim]:
    one balanced collective (every rank sends the same amount), for a dense operand whose rows are
    distributed evenly rather than along the nnz-balanced cuts of A."""
    import torch
    import torch.distributed as dist
    per, dim = x_block.shape
    if out is None:
        out = torch.empty((world_size * per, dim), dtype=x_block.dtype, device=x_block.device)
    if world_size == 1:
        out.copy_(x_block)
        return (out, None) if async_op else out
    work = dist.all_gather_into_tensor(out, x_block.contiguous(), group=group, async_op=async_op)
    return (out, work) if async_op else out


class ShardedSpmm:
    """This rank's shard of a degree-ordered A, ready to multiply.

    indptr / indices / vals are the FULL degree-ordered matrix as CUDA tensors
    on this rank's device (every rank builds the same synthetic matrix from the
    same seed, or loads the same files); the shard is cut out here."""

    def __init__(self, indptr, indices, vals, rank: int, world_size: int, group=None):
        import torch
        from . import partition, spmm
        self.rank, self.world, self.group = rank, world_size, group
        self.n = indptr.numel() - 1
        self.cuts = nnz_balanced_cuts(indptr.cpu().numpy(), world_size)
        ip, ix, v = shard_rows(indptr, indices, vals, self.cuts, rank)
        self.indptr = ip.contiguous()
        self.vals = v.contiguous()
        self.indices = ix.contiguous()
        self.n_local = self.indptr.numel() - 1
        self.n_cols = self.n
        self.block4 = partition.block_level_partition_device(self.indptr)
        self.plan = spmm.SpmmPlan(self.block4, self.indices, self.n_local, self.n_cols)
        self._gather = {}
        self.device = indptr.device
        self._torch = torch

    @property
    def row_range(self):
        return int(self.cuts[self.rank]), int(self.cuts[self.rank + 1])

    def even_block(self, x_full_rows):
        """This rank's block of an evenly distributed dense operand, given a callable or tensor that
        yields rows [a, b) of it; the last rank's block is zero-padded to the common height."""
        per = even_rows(self.n, self.world)
        a, b = min(self.n, self.rank * per), min(self.n, (self.rank + 1) * per)
        rows = x_full_rows(a, b) if callable(x_full_rows) else x_full_rows[a:b]
        if rows.shape[0] == per:
            return rows.contiguous()
        blk = self._torch.zeros((per, rows.shape[1]), dtype=rows.dtype, device=rows.device)
        blk[: rows.shape[0]] = rows
        return blk

    def gather_even_async(self, x_block):
        """Start the balanced all-gather of an evenly distributed operand (see all_gather_even);
        returns (buffer, work).  Column ids index the buffer directly: block r starts at row
        r * rows_per_rank = the global row id of its first row."""
        dim = x_block.shape[1]
        if self.world == 1:
            return x_block, None
        key = ("even", dim)
        buf = self._gather.get(key)
        if buf is None:
            buf = self._torch.empty((self.world * x_block.shape[0], dim), dtype=x_block.dtype, device=self.device)
            self._gather[key] = buf
        return all_gather_even(x_block, self.world, out=buf, group=self.group, async_op=True)

    def gather_async(self, x_local):
        """Start the all-gather of this rank's rows of the dense operand and return (buffer, work).
        The collective runs on the process group's own stream; call work.wait() (it only makes the
        current stream wait) before multiplying.  Gathers of independent operands can therefore be
        in flight while earlier products are still being computed.  One buffer per width."""
        dim = x_local.shape[1]
        if self.world == 1:
            return x_local, None
        buf = self._gather.get(dim)
        if buf is None:
            buf = self._torch.empty((self.n_cols, dim), dtype=x_local.dtype, device=self.device)
            self._gather[dim] = buf
        return all_gather_rows(x_local, self.cuts, self.rank, self.world, out=buf, group=self.group, async_op=True)

    def step(self, x_local, y_local, x_gathered=None):
        """y_local[n_local x dim] = A_shard @ allgather(x_local).  Asynchronous on the current stream.
        x_gathered, if given, is the already gathered [n x dim] operand (the collective is skipped)."""
        dim = y_local.shape[1]
        if x_gathered is not None:
            x_full = x_gathered
        elif self.world == 1:
            x_full = x_local
        else:
            buf = self._gather.get(dim)
            if buf is None:
                buf = self._torch.empty((self.n_cols, dim), dtype=x_local.dtype, device=self.device)
                self._gather[dim] = buf
            x_full = all_gather_rows(x_local, self.cuts, self.rank, self.world, out=buf, group=self.group)
        self.plan.run(self.indices, self.vals, x_full, y_local, dim=dim, ldx=dim, ldy=dim)
        return y_local

    def close(self):
        self.plan.close()
