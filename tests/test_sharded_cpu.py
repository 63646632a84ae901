"""Host-side logic of the row-sharded path on CPU: nnz-balanced cuts, row shards and the
uneven all-gather over the gloo backend with two and three ranks.  The arithmetic of a shard is
checked with the CPU oracle here; the GPU kernels are covered by the -m gpu tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import spmm_close
from oracle import oracle


def _graph(n=700, seed=0):
    rng = np.random.default_rng(seed)
    deg = np.sort(np.minimum((rng.pareto(1.0, n) * 3).astype(np.int64), n // 2))
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    idx = np.concatenate([np.sort(rng.choice(n, d, replace=False)) for d in deg]).astype(np.int32)
    val = rng.random(len(idx)).astype(np.float32)
    return indptr, idx, val


def test_cuts_balance_nonzeros_not_rows():
    from accelgcn import sharded
    indptr, _, _ = _graph(5000, 1)
    for parts in (1, 2, 4, 8):
        cuts = sharded.nnz_balanced_cuts(indptr, parts)
        assert cuts[0] == 0 and cuts[-1] == 5000 and np.all(np.diff(cuts) >= 0) and len(cuts) == parts + 1
        per = np.diff(indptr[cuts].astype(np.int64))
        assert per.sum() == indptr[-1]
        if parts > 1:
            assert per.max() - per.min() <= 2 * np.diff(indptr).max()          # within one (heaviest) row
            assert np.diff(cuts).max() > 2 * np.diff(cuts).min()                # rows are NOT balanced


def test_cuts_degenerate_inputs():
    from accelgcn import sharded
    assert sharded.nnz_balanced_cuts(np.zeros(5, dtype=np.int32), 4).tolist() == [0, 0, 0, 0, 4]
    assert sharded.nnz_balanced_cuts(np.array([0, 10]), 3).tolist()[-1] == 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, dim, result_dir):
    from accelgcn import sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        indptr, idx, val = _graph()
        n = len(indptr) - 1
        x = np.random.default_rng(7).uniform(-1, 1, (n, dim)).astype(np.float32)
        cuts = sharded.nnz_balanced_cuts(indptr, world)
        ip, ix, v = sharded.shard_rows(indptr, idx, val, cuts, rank)
        r0, r1 = int(cuts[rank]), int(cuts[rank + 1])
        x_full = sharded.all_gather_rows(torch.from_numpy(x[r0:r1].copy()), cuts, rank, world).numpy()
        assert np.array_equal(x_full, x)          # uneven blocks land in global row order
        # the evenly distributed operand: one balanced all-gather, rows in global order, tail padded
        per = sharded.even_rows(n, world)
        blk = np.zeros((per, dim), dtype=np.float32)
        a, b = min(n, rank * per), min(n, (rank + 1) * per)
        blk[: b - a] = x[a:b]
        x_even = sharded.all_gather_even(torch.from_numpy(blk), world).numpy()
        assert x_even.shape[0] == world * per and np.array_equal(x_even[:n], x)
        # the shard's own .block4 and product, computed by the oracle (this is a CPU test)
        y = oracle.spmm_block4(oracle.partition(ip), ix, v, x_full, r1 - r0)
        np.save(os.path.join(result_dir, f"y{rank}.npy"), y)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_two_rank_gloo_sharded_product_equals_single_rank(world, tmp_path):
    dim = 12
    mp.spawn(_worker, args=(world, _free_port(), dim, str(tmp_path)), nprocs=world, join=True)
    indptr, idx, val = _graph()
    x = np.random.default_rng(7).uniform(-1, 1, (len(indptr) - 1, dim)).astype(np.float32)
    ref = oracle.spmm_csr(indptr, idx, val, x)
    y = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(world)])
    assert y.shape == ref.shape and spmm_close(y, ref, np.full(len(ref), 50.0)).all()


def _failing_worker(rank, world, port, result_dir):
    # rank 1 leaves between steps (no collective of its own in flight); rank 0 must get an error from
    # its next exchange within the process-group timeout instead of waiting forever
    import datetime
    import time
    from accelgcn import sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    cuts = np.array([0, 3, 6])
    x = torch.ones((3, 4))
    sharded.all_gather_rows(x, cuts, rank, world)            # step 1: everyone is here
    if rank == 1:
        os._exit(0)                                           # gone before step 2
    t0 = time.time()
    try:
        sharded.all_gather_rows(x, cuts, rank, world)
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
