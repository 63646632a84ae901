"""The CPU oracle of the partitioner against the reference's golden vectors (no GPU)."""
import glob
import os

import numpy as np
import pytest

from conftest import kat_indptr, sha256_block4
from oracle import oracle

REFERENCE = oracle.REFERENCE_DIR or ""        # "" when no reference checkout is around: the live tests skip


def test_pattern_tables_closed_form():
    # block_level_partition.py:7-21 against the closed form the kernels use
    warp_nz, rows = oracle.pattern_tables()
    assert len(warp_nz) == len(rows) == 192
    for d in range(1, 192):
        r = 12 if d <= 32 else 6 if d <= 64 else 4 if d <= 96 else 3 if d <= 128 else 2
        f = 12 // r
        assert rows[d] == r and warp_nz[d] == -(-d // f), d


def test_oracle_matches_all_16_golden_block4(kat):
    assert len(kat) == 16
    for name, entry in kat.items():
        got = oracle.partition(kat_indptr(entry))
        assert len(got) == entry["n_blocks"], name
        assert sha256_block4(got) == entry["sha256"], name


def test_python_and_c_oracle_agree_on_small_goldens(kat):
    for name in ("pubmed", "artist", "arxiv"):
        ip = kat_indptr(kat[name])
        assert np.array_equal(oracle.partition_py(ip), oracle.partition(ip)), name


def test_oracle_matches_reference_script_edge_cases(edge_cases):
    assert len(edge_cases) >= 14
    for name, (indptr, want) in edge_cases.items():
        assert np.array_equal(oracle.partition(indptr), want), name
        assert np.array_equal(oracle.partition_py(indptr), want), name


@pytest.mark.skipif(not (REFERENCE and os.path.isdir(os.path.join(REFERENCE, "block_level_meta"))), reason="reference tree not present")
def test_kat_fixture_is_the_reference_files(kat):
    # the committed fixture really is the reference's goldens, byte for byte
    files = sorted(glob.glob(os.path.join(REFERENCE, "block_level_meta", "*.block4")))
    assert len(files) == len(kat)
    for f in files:
        name = os.path.basename(f)[: -len(".block4")]
        raw = np.fromfile(f, dtype=np.int32).reshape(-1, 4)
        assert np.array_equal(oracle.partition(kat_indptr(kat[name])), raw), name


def test_empty_graph_raises():
    with pytest.raises(IndexError):
        oracle.partition_py(np.array([0], dtype=np.int32))
    with pytest.raises(ValueError):
        oracle.partition(np.array([0], dtype=np.int32))


def test_degree_sort_oracle_properties():
    rng = np.random.default_rng(3)
    deg = rng.integers(0, 9, 200)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    idx = rng.integers(0, 200, indptr[-1]).astype(np.int32)
    val = rng.random(indptr[-1]).astype(np.float32)
    perm, nip, nidx, nval = oracle.degree_sort(indptr, idx, val, relabel_cols=True)
    nd = np.diff(nip)
    assert np.all(np.diff(nd) >= 0) and sorted(perm) == list(range(200))
    # stable: equal degrees keep ascending original ids
    for d in np.unique(nd):
        assert np.all(np.diff(perm[nd == d]) > 0)
    # row r of the new matrix is row perm[r] of the old one, columns renamed
    inv = np.empty(200, dtype=np.int64); inv[perm] = np.arange(200)
    for r in (0, 57, 199):
        o = perm[r]
        assert np.array_equal(nidx[nip[r]:nip[r + 1]], inv[idx[indptr[o]:indptr[o + 1]]])
        assert np.array_equal(nval[nip[r]:nip[r + 1]], val[indptr[o]:indptr[o + 1]])


@pytest.mark.skipif(not (REFERENCE and os.path.isfile(os.path.join(REFERENCE, "block_level_partition.py"))), reason="reference tree not present")
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_oracle_against_the_unmodified_script_run_live(seed, tmp_path):
    # fresh random degree sequences through the reference script itself (subprocess, scratch directory
    # laid out as it expects), not only the committed fixtures
    import subprocess
    import sys
    rng = np.random.default_rng(1000 + seed)
    cases = {
        "sorted": np.sort(rng.choice(np.array([0, 1, 2, 3, 30, 32, 33, 64, 65, 96, 97, 128, 129, 191, 192, 384, 385, 800]), 3000)),
        "unsorted": rng.choice(np.array([0, 1, 1, 2, 12, 33, 100, 191, 192, 400, 1200]), 3000),
        "runs": np.repeat(rng.integers(1, 200, 200), rng.integers(1, 30, 200)),
    }
    os.makedirs(tmp_path / "graphs")
    for name, deg in cases.items():
        indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
        (tmp_path / "graphs" / f"{name}.config").write_text("")
        indptr.tofile(tmp_path / "graphs" / f"{name}.new_indptr")
        np.zeros(int(indptr[-1]), dtype=np.int32).tofile(tmp_path / "graphs" / f"{name}.new_indices")
    subprocess.check_call([sys.executable, os.path.join(REFERENCE, "block_level_partition.py")], cwd=tmp_path,
                          stdout=subprocess.DEVNULL)
    for name, deg in cases.items():
        want = np.fromfile(tmp_path / "block_level_meta" / f"{name}.block4", dtype=np.int32).reshape(-1, 4)
        indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
        assert np.array_equal(oracle.partition(indptr), want), name
