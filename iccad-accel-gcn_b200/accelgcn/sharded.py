"""1D row-sharded multi-GPU SpMM: one process per GPU; the layout, the exchange (NCCL, inside
libaccelgcn.so) and every kernel are the library's (agcn_dist_*).  This module only owns the
tensors and hands the 128-byte communicator id from rank 0 to the others.

Layout.  Every rank holds two ranges of the degree-ordered rows, one from the light and one
from the heavy end, chosen so that it has rows_per_block rows AND about nnz / world nonzeros
(agcn_balanced_blocks).  Dense operands are "block rows": [rows_per_block x dim] per rank,
padding rows zero; the all-gather of equal blocks is one balanced collective, and the gathered
operand is a permutation of the degree order that the block's column ids were renamed to.

The reference has no multi-GPU code; this follows its single-GPU operator (spmm_accel.cu)
block by block.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib


def balanced_blocks(indptr, world: int):
    """Row ranges of every rank: (ranges int64 [world, 4] = light_begin, light_end, heavy_begin,
    heavy_end; rows_per_block).  Host arrays only -- needs no GPU."""
    lib = _lib.load()
    indptr = np.ascontiguousarray(indptr, dtype=np.int32)
    n = indptr.shape[0] - 1
    ranges = np.zeros((world, 4), dtype=np.int64)
    per = ctypes.c_int64(0)
    _lib.check(lib.agcn_balanced_blocks(indptr.ctypes.data, n, world, ranges.ctypes.data, ctypes.byref(per)))
    return ranges, per.value


def block_rows(ranges, rows_per_block: int, rank: int) -> np.ndarray:
    """Matrix row held at each local row of `rank` (-1 = padding): light rows, heavy rows, padding."""
    la, lb, ha, hb = (int(v) for v in ranges[rank])
    rows = np.concatenate([np.arange(la, lb), np.arange(ha, hb)]).astype(np.int64)
    return np.concatenate([rows, np.full(rows_per_block - len(rows), -1, dtype=np.int64)])


def gathered_position(rows_per_block: int, world: int, slices: int, rank: int) -> np.ndarray:
    """Row of the gathered operand that holds each local row of `rank`'s block.  The operand is
    exchanged in `slices` row slices: slice c of every rank comes first, then slice c + 1, ..."""
    per = rows_per_block
    assert per % slices == 0
    bc = per // slices
    j = np.arange(per, dtype=np.int64)
    c, i = j // bc, j % bc
    return c * (world * bc) + rank * bc + i


def shard_csr(indptr, indices, vals, ranges, rows_per_block: int, world: int, slices: int, rank: int):
    """Host restatement of what agcn_dist_set_graph builds on the device: the block's row pointers,
    column ids renamed to gathered positions, values.  Used by the CPU tests with the oracle."""
    indptr = np.asarray(indptr, dtype=np.int64)
    rows = block_rows(ranges, rows_per_block, rank)
    valid = rows[rows >= 0]
    deg = np.zeros(rows_per_block, dtype=np.int64)
    deg[: len(valid)] = indptr[valid + 1] - indptr[valid]
    ip = np.concatenate([[0], np.cumsum(deg)])
    src = np.concatenate([np.arange(indptr[r], indptr[r + 1]) for r in valid] + [np.zeros(0, dtype=np.int64)]).astype(np.int64)
    new_id = np.full(int(indptr.shape[0] - 1), -1, dtype=np.int64)
    for g in range(world):
        rg = block_rows(ranges, rows_per_block, g)
        pos = gathered_position(rows_per_block, world, slices, g)
        new_id[rg[rg >= 0]] = pos[rg >= 0]
    return ip.astype(np.int32), new_id[np.asarray(indices)[src]].astype(np.int32), np.asarray(vals)[src]


def exchange_id(rank: int, world: int, group=None) -> bytes | None:
    """The communicator id: made by rank 0 inside the library, handed to the other ranks through
    torch.distributed (any transport would do: it is 128 opaque bytes)."""
    if world == 1:
        return None
    import torch.distributed as dist
    box = [None]
    if rank == 0:
        buf = ctypes.create_string_buffer(_lib.DIST_ID_BYTES)
        _lib.check(_lib.load().agcn_dist_unique_id(buf))
        box[0] = bytes(buf.raw)
    src = dist.get_global_rank(group, 0) if group is not None else 0
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]


def feature_groups(rank: int, world: int, groups: int):
    """Rows x features decomposition of a product that is wide enough: the ranks form `groups` feature
    groups; group j multiplies columns [j * dim / groups, (j + 1) * dim / groups) of the dense operand
    on a row-sharded A over its own world / groups ranks, with its own communicator.  Every exchange
    then moves 1 / groups of the columns among world / groups ranks, and a rank's block of A has
    groups times the rows at 1 / groups of the width.  Returns (row_rank, row_world, feature_group,
    ranks of this rank's communicator); rank = row_rank * groups + feature_group."""
    assert groups >= 1 and world % groups == 0, "the number of feature groups must divide the number of ranks"
    j = rank % groups
    return rank // groups, world // groups, j, list(range(j, world, groups))


class ShardedSpmm:
    """This rank's block of a degree-ordered square A, ready to multiply.

    indptr / indices / vals are the WHOLE degree-ordered matrix as CUDA tensors on this rank's
    device (every rank builds the same synthetic matrix from the same seed, or loads the same
    files); the block is cut out inside the library.  `exchange_slices` > 1 exchanges the dense
    operand in that many row slices and starts the product over a slice when it has arrived;
    `column_ranges` > 1 (with one slice) tiles the block's columns for a gathered operand larger than L2.
    `communicator=False` builds the block without NCCL (the caller assembles the gathered operand
    itself and calls `multiply_gathered`): used to run every rank's block in one process."""

    def __init__(self, indptr, indices, vals, rank: int, world_size: int, group=None, exchange_slices: int = 1,
                 communicator: bool = True, column_ranges: int = 1):
        import torch
        self._torch = torch
        self._lib = lib = _lib.load()
        self.rank, self.world, self.group = int(rank), int(world_size), group
        self.device = indptr.device
        self.n = int(indptr.numel()) - 1
        uid = exchange_id(self.rank, self.world, group) if communicator else None
        h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(lib.agcn_dist_create(ctypes.byref(h), self.rank, self.world, uid))
            self._h = h
            s = torch.cuda.current_stream(self.device)
            _lib.check(lib.agcn_dist_set_graph(h, indptr.data_ptr(), indices.data_ptr(), vals.data_ptr(), self.n,
                                               int(indices.numel()), int(exchange_slices), int(column_ranges), s.cuda_stream))
        info = self.info()
        self.rows_per_block, self.slices = info["rows_per_block"], info["exchange_slices"]
        self.local_rows, self.local_nnz, self.n_blocks = info["local_rows"], info["local_nnz"], info["n_blocks"]
        self.n_gathered = self.rows_per_block * self.world
        self._rows = {}

    def info(self) -> dict:
        a, b, c, d = (ctypes.c_int64() for _ in range(4))
        e, f = ctypes.c_int(), ctypes.c_int()
        _lib.check(self._lib.agcn_dist_info(self._h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), ctypes.byref(d),
                                            ctypes.byref(e), ctypes.byref(f)))
        return {"rows_per_block": a.value, "local_rows": b.value, "local_nnz": c.value, "n_blocks": d.value,
                "exchange_slices": e.value, "launches_last_step": f.value}

    def rows_of(self, rank: int | None = None):
        """int64 CUDA tensor [rows_per_block]: the matrix row at each local row of `rank` (-1 = padding)."""
        torch = self._torch
        rank = self.rank if rank is None else rank
        if rank not in self._rows:
            out = torch.empty(self.rows_per_block, dtype=torch.int32, device=self.device)
            with torch.cuda.device(self.device):
                _lib.check(self._lib.agcn_dist_block_rows(self._h, rank, out.data_ptr(),
                                                          torch.cuda.current_stream(self.device).cuda_stream))
            self._rows[rank] = out.to(torch.int64)
        return self._rows[rank]

    def to_block(self, x_rows):
        """This rank's block rows [rows_per_block x dim] of a dense operand given in matrix order:
        x_rows is a tensor [n x dim] or a callable rows -> tensor (for operands too large to build whole)."""
        torch = self._torch
        rows = self.rows_of()
        valid = rows >= 0
        picked = x_rows(rows[valid]) if callable(x_rows) else x_rows[rows[valid]]
        blk = torch.zeros((self.rows_per_block, picked.shape[1]), dtype=torch.float32, device=self.device)
        blk[valid] = picked
        return blk

    def from_blocks(self, blocks):
        """Matrix-order [n x dim] tensor from the block rows of every rank (tests, single process)."""
        torch = self._torch
        out = torch.empty((self.n, blocks[0].shape[1]), dtype=torch.float32, device=self.device)
        for g, blk in enumerate(blocks):
            rows = self.rows_of(g)
            out[rows[rows >= 0]] = blk[rows >= 0]
        return out

    def _stream(self, stream):
        return (stream if stream is not None else self._torch.cuda.current_stream(self.device)).cuda_stream

    def gather_begin(self, x_block, slot: int = 0, stream=None) -> None:
        """Start the all-gather of this rank's block into `slot` (0..3), behind the work already on
        the stream.  Exchanges of independent products can be started together."""
        rc = self._lib.agcn_dist_gather_begin(self._h, slot, x_block.data_ptr(), int(x_block.shape[1]), self._stream(stream))
        if rc != 0:
            _lib.check(rc)

    def multiply(self, y_block, slot: int = 0, relu: bool = False, stream=None) -> None:
        """y_block = act(A_block @ gathered operand of `slot`); the stream waits for the exchange slice by slice."""
        rc = self._lib.agcn_dist_spmm_gathered(self._h, slot, y_block.data_ptr(), int(y_block.shape[1]), 1 if relu else 0,
                                               self._stream(stream))
        if rc != 0:
            _lib.check(rc)

    def wait_gathered(self, slot: int = 0, stream=None) -> None:
        """Make the stream wait for the whole exchange of `slot` without multiplying."""
        _lib.check(self._lib.agcn_dist_wait_gathered(self._h, slot, self._stream(stream)))

    def step(self, x_block, y_block, relu: bool = False, stream=None):
        """One product: all-gather x_block, then y_block = act(A_block @ X).  Asynchronous."""
        rc = self._lib.agcn_dist_spmm_step(self._h, x_block.data_ptr(), y_block.data_ptr(), int(y_block.shape[1]),
                                           1 if relu else 0, self._stream(stream))
        if rc != 0:
            _lib.check(rc)
        return y_block

    def multiply_gathered(self, gathered, y_block, relu: bool = False, stream=None):
        """The local product on a gathered operand [world * rows_per_block x dim] assembled by the caller."""
        _lib.check(self._lib.agcn_dist_spmm_on_gathered(self._h, gathered.data_ptr(), y_block.data_ptr(), int(y_block.shape[1]),
                                                        1 if relu else 0, self._stream(stream)))
        return y_block

    def assemble_gathered(self, blocks):
        """What the all-gather produces from every rank's block (tests, single process)."""
        torch = self._torch
        dim = blocks[0].shape[1]
        out = torch.empty((self.n_gathered, dim), dtype=torch.float32, device=self.device)
        for g, blk in enumerate(blocks):
            pos = torch.from_numpy(gathered_position(self.rows_per_block, self.world, self.slices, g)).to(self.device)
            out[pos] = blk
        return out

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.agcn_dist_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
