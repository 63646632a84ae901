"""Regenerates the fixtures in this directory.  Needs the reference source tree
(its location is oracle.REFERENCE_DIR, settable with ACCELGCN_REFERENCE); the
tests themselves only read the committed fixtures.

    python tests/golden/make_golden.py

1. block4_kat.json -- known-answer vectors for the partitioner.  Each of the
   16 ``block_level_meta/<graph>.block4`` files the reference ships is
   inverted to the degree sequence it was made from (leading zero-degree rows
   + run-length-encoded ascending degrees) and stored with the SHA-256 and
   block count of the golden file.  A partitioner is right iff, fed that
   degree sequence, it reproduces a file with that hash.
2. partition_edge_cases.npz -- seeded edge-case inputs (unsorted degrees,
   zero-degree rows anywhere, every pattern boundary, heavy rows) with the
   outputs of the UNMODIFIED reference script block_level_partition.py, run
   here through ``subprocess`` in a scratch directory laid out as the script
   expects (./graphs/<g>.config, .new_indptr, .new_indices -> ./block_level_meta/).
"""
import glob
import hashlib
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.oracle import REFERENCE_DIR as REF  # noqa: E402

if REF is None:
    sys.exit("make_golden.py needs the reference checkout: set ACCELGCN_REFERENCE=/path/to/ICCAD-Accel-GCN")


def invert_block4(b):
    """.block4 tuples -> (leading zero rows, degrees[], counts[]) of the sorted degree sequence."""
    deg, row, _loc, info = b.T
    small = deg <= 384
    first = np.ones(len(b), bool)
    first[1:] = ~((~small[1:]) & (row[1:] == row[:-1]))
    rows_per_entry = np.where(small, info & 0xFFFF, first.astype(np.int32))
    degs = np.repeat(deg, rows_per_entry)
    change = np.flatnonzero(np.diff(degs)) + 1
    starts = np.concatenate([[0], change])
    counts = np.diff(np.concatenate([starts, [len(degs)]]))
    return int(row[0]), degs[starts].tolist(), counts.tolist()


def make_kat():
    kat = {}
    for f in sorted(glob.glob(os.path.join(REF, "block_level_meta", "*.block4"))):
        raw = open(f, "rb").read()
        b = np.frombuffer(raw, dtype=np.int32).reshape(-1, 4)
        lead, d, c = invert_block4(b)
        kat[os.path.basename(f)[:-len(".block4")]] = {
            "leading_zero_rows": lead, "degrees": d, "counts": c,
            "n_blocks": int(len(b)), "sha256": hashlib.sha256(raw).hexdigest(),
        }
    with open(os.path.join(HERE, "block4_kat.json"), "w") as fh:
        json.dump(kat, fh, separators=(",", ":"))
    print("block4_kat.json:", len(kat), "graphs")


def edge_case_degrees():
    rng = np.random.default_rng(20231)
    cases = {}
    boundary = [1, 2, 31, 32, 33, 63, 64, 65, 95, 96, 97, 127, 128, 129, 190, 191, 192, 193,
                383, 384, 385, 767, 768, 769, 1152, 1153, 5000]
    cases["single_row_deg1"] = np.array([1])
    cases["single_row_heavy"] = np.array([1000])
    # (graphs with no nonzero at all make the script raise inside scipy's csr_matrix, so none is listed)
    cases["all_zero_but_last"] = np.concatenate([np.zeros(7, dtype=np.int64), [2]])
    cases["boundaries_once"] = np.array(boundary)
    cases["boundaries_runs"] = np.repeat(np.array(boundary), rng.integers(1, 30, len(boundary)))
    cases["trailing_zeros"] = np.concatenate([np.sort(rng.integers(0, 50, 300)), np.zeros(11, dtype=np.int64)])
    cases["interior_zeros_unsorted"] = rng.choice(np.array([0, 0, 1, 1, 2, 5, 5, 33, 100, 400]), 500)
    cases["unsorted_random"] = rng.integers(0, 420, 2000)
    cases["unsorted_boundary_mix"] = rng.choice(np.array(boundary + [0, 0]), 1500)
    cases["long_runs"] = np.concatenate([np.full(1000, 1), np.full(777, 3), np.full(100, 32), np.full(50, 33),
                                         np.full(25, 192), np.full(7, 385)])
    cases["run_lengths_mod_rows"] = np.concatenate([np.full(k, d) for d in (1, 40, 70, 100, 150)
                                                    for k in (1, 2, 3, 4, 5, 6, 7, 11, 12, 13, 24, 25)
                                                    for _ in (0,)] )
    # alternate so equal-degree runs are split by a different degree between them
    alt = []
    for k in range(1, 30):
        alt += [2] * k + [3]
    cases["alternating_runs"] = np.array(alt)
    w = rng.pareto(1.1, 4000) + 1
    cases["sorted_power_law"] = np.sort(np.minimum((w * 3).astype(np.int64), 20000))
    cases["sorted_with_leading_zeros"] = np.sort(np.concatenate([np.zeros(123, dtype=np.int64), rng.integers(1, 600, 900)]))
    return {k: np.asarray(v, dtype=np.int64) for k, v in cases.items()}


def run_reference_script(cases):
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        os.makedirs(os.path.join(tmp, "graphs"))
        for name, deg in cases.items():
            indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
            nnz = int(indptr[-1])
            open(os.path.join(tmp, "graphs", name + ".config"), "w").close()
            indptr.tofile(os.path.join(tmp, "graphs", name + ".new_indptr"))
            np.zeros(nnz, dtype=np.int32).tofile(os.path.join(tmp, "graphs", name + ".new_indices"))
        subprocess.check_call([sys.executable, os.path.join(REF, "block_level_partition.py")], cwd=tmp,
                              stdout=subprocess.DEVNULL)
        for name in cases:
            out[name] = np.fromfile(os.path.join(tmp, "block_level_meta", name + ".block4"), dtype=np.int32)
    return out


def make_edge_cases():
    cases = edge_case_degrees()
    got = run_reference_script(cases)
    blob = {}
    for name, deg in cases.items():
        blob["indptr__" + name] = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
        blob["block4__" + name] = got[name]
    np.savez_compressed(os.path.join(HERE, "partition_edge_cases.npz"), **blob)
    print("partition_edge_cases.npz:", len(cases), "cases,",
          sum(len(v) // 4 for v in got.values()), "blocks")


if __name__ == "__main__":
    make_kat()
    make_edge_cases()
