"""Parity of the GPU partitioner with the oracle / reference goldens, through the C ABI."""
import ctypes

import numpy as np
import pytest

from conftest import kat_indptr, sha256_block4, require_cuda
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_golden_block4_files_bit_exact_host_entry(kat):
    from accelgcn import partition
    require_cuda()
    for name, entry in kat.items():
        got = partition.block_level_partition(kat_indptr(entry))
        assert len(got) == entry["n_blocks"], name
        assert sha256_block4(got) == entry["sha256"], name


def test_golden_block4_files_bit_exact_device_entry(kat):
    import torch
    from accelgcn import partition
    dev = require_cuda()
    for name in ("pubmed", "am", "citation", "ppa", "arxiv", "youtube"):
        ip = torch.from_numpy(kat_indptr(kat[name])).to(dev)
        got = partition.block_level_partition_device(ip).cpu().numpy()
        assert sha256_block4(got) == kat[name]["sha256"], name


def test_reference_script_edge_cases_bit_exact(edge_cases):
    from accelgcn import partition
    require_cuda()
    for name, (indptr, want) in edge_cases.items():
        got = partition.block_level_partition(indptr)
        assert np.array_equal(got, want), name


@pytest.mark.parametrize("seed", range(8))
def test_random_degree_sequences_match_oracle(seed):
    from accelgcn import partition
    require_cuda()
    rng = np.random.default_rng(seed)
    n = int(rng.integers(1, 200_000))
    pool = np.array([0, 0, 1, 1, 1, 2, 3, 12, 31, 32, 33, 64, 65, 96, 97, 128, 129, 191, 192, 383, 384, 385, 769, 4000])
    if seed % 2:
        deg = rng.choice(pool, n)                         # unsorted, many short runs
    else:
        deg = np.sort(rng.choice(pool, n))                # sorted, long runs crossing many tiles
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    assert np.array_equal(partition.block_level_partition(indptr), oracle.partition(indptr))


def test_nonzero_first_pointer_and_all_zero_degrees():
    from accelgcn import partition
    require_cuda()
    deg = np.array([3, 3, 3, 0, 500])
    ip = (np.concatenate([[0], np.cumsum(deg)]) + 17).astype(np.int32)
    assert np.array_equal(partition.block_level_partition(ip), oracle.partition(ip - 17))
    # a graph with rows but no nonzero: no tuples (the reference script fails inside scipy here)
    assert partition.block_level_partition(np.zeros(9, dtype=np.int32)).shape == (0, 4)


def test_full_size_degree_sequence_matches_oracle_and_invariants():
    # 5 million rows with the degree mix of the large configurations: bit-exact against the C
    # oracle, plus format invariants that hold at any size
    from accelgcn import partition
    require_cuda()
    rng = np.random.default_rng(99)
    n = 5_000_000
    deg = np.sort(np.minimum((rng.pareto(1.2, n) * 6).astype(np.int64), 20_000))
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    got = partition.block_level_partition(indptr)
    assert np.array_equal(got, oracle.partition(indptr))
    d, row, loc, info = got.T.astype(np.int64)
    small = d <= 384
    nz = np.where(small, (info & 0xFFFF) * d, info)
    assert nz.sum() == indptr[-1] and np.all(nz <= 384)
    assert np.array_equal(loc, np.concatenate([[0], np.cumsum(nz)[:-1]]))        # tuples tile the nonzeros
    assert np.array_equal(loc[small], indptr[row[small]])


def test_error_behaviour():
    from accelgcn import _lib
    require_cuda()
    lib = _lib.load()
    n = ctypes.c_int64(0)
    bad = np.array([0, 5, 3, 9], dtype=np.int32)                                  # negative degree
    assert lib.agcn_partition_host(bad.ctypes.data, 3, None, 0, ctypes.byref(n)) == _lib.ERR_RANGE
    ip = np.array([0, 1, 2, 1000], dtype=np.int32)
    out = np.zeros((2, 4), dtype=np.int32)
    assert lib.agcn_partition_host(ip.ctypes.data, 3, out.ctypes.data, 2, ctypes.byref(n)) == _lib.ERR_CAPACITY
    assert n.value == 4                                                           # 1 + ceil(998 / 384)


def test_drop_in_script_same_files_as_the_reference(kat, tmp_path):
    # run like the reference script: cwd holding ./graphs/<g>.config + .new_indptr -> ./block_level_meta/<g>.block4
    import subprocess, sys, os
    from conftest import PKG
    require_cuda()
    os.makedirs(tmp_path / "graphs")
    for name in ("pubmed", "collab"):
        (tmp_path / "graphs" / f"{name}.config").write_text("")
        kat_indptr(kat[name]).tofile(tmp_path / "graphs" / f"{name}.new_indptr")
    subprocess.check_call([sys.executable, os.path.join(PKG, "block_level_partition.py")], cwd=tmp_path,
                          stdout=subprocess.DEVNULL)
    for name in ("pubmed", "collab"):
        got = np.fromfile(tmp_path / "block_level_meta" / f"{name}.block4", dtype=np.int32)
        assert sha256_block4(got) == kat[name]["sha256"], name
