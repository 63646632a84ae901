"""Drop-in replacement of the reference's block_level_partition.py: same invocation, same files.

Run from a directory that holds ./graphs/ (as the reference script is run from its repository
root, README.md:54-58).  For every ./graphs/<g>.config it reads ./graphs/<g>.new_indptr (int32,
degree-ordered row pointers; block_level_partition.py:31) and writes ./block_level_meta/<g>.block4
(:105-106) -- byte-identical to the reference's output, computed on the GPU through the C ABI
(agcn_partition_host).  There is no CPU fallback.
"""
import os
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from accelgcn import graphio, partition  # noqa: E402


def main(base_path="./graphs/", out_path="./block_level_meta/"):
    os.makedirs(out_path, exist_ok=True)
    for file in Path(base_path).glob("*.config"):          # the .config content is never read (:26-29)
        print(file.stem)
        new_indptr = np.fromfile(os.path.join(base_path, file.stem + ".new_indptr"), dtype=np.int32)
        v_num, e_num = len(new_indptr) - 1, int(new_indptr[-1]) if len(new_indptr) else 0
        print(v_num, e_num)
        graphio.write_block4(os.path.join(out_path, file.stem + ".block4"),
                             partition.block_level_partition(new_indptr))


if __name__ == "__main__":
    main()
