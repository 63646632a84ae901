"""Host-side logic of the row-sharded path on CPU: the balanced two-range row blocks
(agcn_balanced_blocks is host code and needs no GPU), the renaming of column ids to gathered
positions, and the balanced all-gather over the gloo backend with two, three and four ranks.
The arithmetic of a block is checked with the CPU oracle here; the GPU kernels and the NCCL
exchange are covered by the -m gpu tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import spmm_close
from oracle import oracle


def _graph(n=700, seed=0, hub=0):
    rng = np.random.default_rng(seed)
    deg = np.sort(np.minimum((rng.pareto(1.0, n) * 3).astype(np.int64), n // 2))
    if hub:
        deg[-1] = hub                       # one row with most of the nonzeros
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    idx = np.concatenate([np.sort(rng.choice(n, d, replace=False)) for d in deg]).astype(np.int32)
    val = rng.random(len(idx)).astype(np.float32)
    return indptr, idx, val


def test_blocks_balance_rows_and_nonzeros():
    from accelgcn import sharded
    indptr, _, _ = _graph(5000, 1)
    deg = np.diff(indptr.astype(np.int64))
    for world in (1, 2, 4, 8):
        ranges, per = sharded.balanced_blocks(indptr, world)
        assert per == -(-5000 // world) and ranges.shape == (world, 4)
        rows = [sharded.block_rows(ranges, per, g) for g in range(world)]
        owned = np.concatenate([r[r >= 0] for r in rows])
        assert len(owned) == 5000 and np.array_equal(np.sort(owned), np.arange(5000))      # a partition of the rows
        nnz = np.array([deg[r[r >= 0]].sum() for r in rows])
        assert nnz.sum() == indptr[-1]
        if world > 1:
            assert nnz.max() - nnz.min() <= 2 * deg.max()                 # within one (heaviest) row of each other
            assert max(len(r[r >= 0]) for r in rows) - min(len(r[r >= 0]) for r in rows) <= world     # rows balanced too
        for r in rows:                                                     # ascending degree inside a block
            assert np.all(np.diff(deg[r[r >= 0]]) >= 0)


def test_blocks_degenerate_inputs():
    from accelgcn import sharded, AccelGcnError
    ranges, per = sharded.balanced_blocks(np.zeros(6, dtype=np.int32), 4)          # 5 rows, no nonzeros
    assert per == 2 and sorted(np.concatenate([sharded.block_rows(ranges, per, g) for g in range(4)]).tolist()) == [-1, -1, -1, 0, 1, 2, 3, 4]
    ranges, per = sharded.balanced_blocks(np.array([0, 10], dtype=np.int32), 3)    # fewer rows than ranks: empty blocks
    assert per == 1 and [int((sharded.block_rows(ranges, per, g) >= 0).sum()) for g in range(3)] == [1, 0, 0]
    with pytest.raises(AccelGcnError):
        sharded.balanced_blocks(np.array([0, 1], dtype=np.int32), 0)
    # a hub row holding most of the nonzeros: every rank still gets its share of rows (no empty shard)
    indptr, _, _ = _graph(400, 3, hub=190)
    ranges, per = sharded.balanced_blocks(indptr, 8)
    assert all(int((sharded.block_rows(ranges, per, g) >= 0).sum()) == 50 for g in range(8))


def test_gathered_positions_tile_the_operand():
    from accelgcn import sharded
    for world, per, slices in ((3, 12, 1), (4, 12, 3), (2, 8, 4)):
        pos = np.concatenate([sharded.gathered_position(per, world, slices, g) for g in range(world)])
        assert np.array_equal(np.sort(pos), np.arange(world * per))
        # slice c of every rank is contiguous: what one all-gather of that slice writes
        bc = per // slices
        for g in range(world):
            p = sharded.gathered_position(per, world, slices, g)
            for c in range(slices):
                assert np.array_equal(p[c * bc:(c + 1) * bc], np.arange(bc) + c * world * bc + g * bc)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, dim, slices, hub, result_dir):
    from accelgcn import sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        indptr, idx, val = _graph(hub=hub)
        n = len(indptr) - 1
        x = np.random.default_rng(7).uniform(-1, 1, (n, dim)).astype(np.float32)
        ranges, per = sharded.balanced_blocks(indptr, world)
        per = -(-per // slices) * slices
        rows = sharded.block_rows(ranges, per, rank)
        blk = np.zeros((per, dim), dtype=np.float32)
        blk[rows >= 0] = x[rows[rows >= 0]]
        # the exchange: one balanced all-gather per slice, each into its contiguous region
        bc = per // slices
        gathered = torch.zeros((world * per, dim))
        for c in range(slices):
            dist.all_gather_into_tensor(gathered[c * world * bc:(c + 1) * world * bc], torch.from_numpy(blk[c * bc:(c + 1) * bc].copy()))
        gathered = gathered.numpy()
        pos = sharded.gathered_position(per, world, slices, rank)
        assert np.array_equal(gathered[pos], blk)
        # this rank's block of A with renamed columns, multiplied by the oracle (this is a CPU test)
        ip, ix, v = sharded.shard_csr(indptr, idx, val, ranges, per, world, slices, rank)
        y = oracle.spmm_block4(oracle.partition(ip), ix, v, gathered, per)
        np.save(os.path.join(result_dir, f"y{rank}.npy"), y)
        np.save(os.path.join(result_dir, f"rows{rank}.npy"), rows)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,slices,hub", [(2, 1, 0), (3, 2, 0), (4, 1, 300)])
def test_gloo_sharded_product_equals_single_rank(world, slices, hub, tmp_path):
    dim = 12
    mp.spawn(_worker, args=(world, _free_port(), dim, slices, hub, str(tmp_path)), nprocs=world, join=True)
    indptr, idx, val = _graph(hub=hub)
    x = np.random.default_rng(7).uniform(-1, 1, (len(indptr) - 1, dim)).astype(np.float32)
    ref = oracle.spmm_csr(indptr, idx, val, x)
    y = np.full_like(ref, np.nan)
    for r in range(world):
        rows, yb = np.load(tmp_path / f"rows{r}.npy"), np.load(tmp_path / f"y{r}.npy")
        y[rows[rows >= 0]] = yb[rows >= 0]
        assert np.all(yb[rows < 0] == 0)                    # padding rows multiply to zero
    assert not np.isnan(y).any() and spmm_close(y, ref, np.full(len(ref), 50.0)).all()


def _feature_group_worker(rank, world, port, dim, groups, result_dir):
    from accelgcn import sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        row_rank, row_world, fgroup, members = sharded.feature_groups(rank, world, groups)
        assert rank == row_rank * groups + fgroup and members[row_rank] == rank
        comms = [dist.new_group(ranks=list(range(j, world, groups))) for j in range(groups)]   # every rank makes every group
        indptr, idx, val = _graph()
        n, w = len(indptr) - 1, dim // groups
        x = np.random.default_rng(7).uniform(-1, 1, (n, dim)).astype(np.float32)[:, fgroup * w:(fgroup + 1) * w]
        ranges, per = sharded.balanced_blocks(indptr, row_world)
        rows = sharded.block_rows(ranges, per, row_rank)
        blk = np.zeros((per, w), dtype=np.float32)
        blk[rows >= 0] = x[rows[rows >= 0]]
        gathered = torch.zeros((row_world * per, w))
        dist.all_gather_into_tensor(gathered, torch.from_numpy(blk), group=comms[fgroup])   # among this group's ranks only
        ip, ix, v = sharded.shard_csr(indptr, idx, val, ranges, per, row_world, 1, row_rank)
        y = oracle.spmm_block4(oracle.partition(ip), ix, v, gathered.numpy(), per)
        np.save(os.path.join(result_dir, f"y{rank}.npy"), y)
        np.save(os.path.join(result_dir, f"rows{rank}.npy"), rows)
    finally:
        dist.destroy_process_group()


def test_gloo_rows_by_features_product_equals_single_rank(tmp_path):
    """4 ranks as 2 feature groups x 2 row ranks: each group multiplies its half of the columns on a
    2-way row-sharded A with its own communicator; the blocks tile Y by rows and columns."""
    world, groups, dim = 4, 2, 12
    mp.spawn(_feature_group_worker, args=(world, _free_port(), dim, groups, str(tmp_path)), nprocs=world, join=True)
    indptr, idx, val = _graph()
    x = np.random.default_rng(7).uniform(-1, 1, (len(indptr) - 1, dim)).astype(np.float32)
    ref = oracle.spmm_csr(indptr, idx, val, x)
    y = np.full_like(ref, np.nan)
    w = dim // groups
    for r in range(world):
        rows, yb = np.load(tmp_path / f"rows{r}.npy"), np.load(tmp_path / f"y{r}.npy")
        j = r % groups
        y[rows[rows >= 0], j * w:(j + 1) * w] = yb[rows >= 0]
    assert not np.isnan(y).any() and spmm_close(y, ref, np.full(len(ref), 50.0)).all()


def _failing_worker(rank, world, port, result_dir):
    # rank 1 leaves between steps (no collective of its own in flight); rank 0 must get an error from
    # its next exchange within the process-group timeout instead of waiting forever
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    blk, out = torch.ones((3, 4)), torch.zeros((6, 4))
    dist.all_gather_into_tensor(out, blk)                    # step 1: everyone is here
    if rank == 1:
        os._exit(0)                                           # gone before step 2
    t0 = time.time()
    try:
        dist.all_gather_into_tensor(out, blk)
        outcome = "no error"
    except Exception as e:                                    # noqa: BLE001
        outcome = f"error after {time.time() - t0:.1f}s: {type(e).__name__}"
    with open(os.path.join(result_dir, "outcome.txt"), "w") as fh:
        fh.write(outcome)
    os._exit(0)


def test_a_rank_that_left_turns_the_next_exchange_into_an_error_not_a_hang(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank is still waiting: the exchange hung"
    outcome = (tmp_path / "outcome.txt").read_text()
    assert outcome.startswith("error after"), outcome
