"""The reference's on-disk formats: headerless little-endian raw arrays.

  graphs/<g>.config                       only enumerated, never read (main.cu:197-215)
  graphs/<g>.new_indptr / .new_indices    degree-ordered CSR, int32 (main.cu:62-63)
  graphs/<g>.graph.ptrdump / .edgedump    CSR in the original order, int32 (main.cu:64-65)
  block_level_meta/<g>.block4             int32 4-tuples (block_level_partition.py:105-106)

Sizes are 64-bit here (the reference's reader keeps the byte length in an int,
data.h:11, and cannot load files of 2 GiB or more).
"""
from __future__ import annotations

import os

import numpy as np


def read_array(path: str, dtype=np.int32) -> np.ndarray:
    size = os.path.getsize(path)
    item = np.dtype(dtype).itemsize
    if size % item:
        raise ValueError(f"{path}: {size} bytes is not a whole number of {np.dtype(dtype).name} items")
    return np.fromfile(path, dtype=dtype)


def write_array(path: str, arr, dtype=np.int32) -> None:
    np.ascontiguousarray(arr, dtype=dtype).tofile(path)


def read_block4(path: str) -> np.ndarray:
    a = read_array(path, np.int32)
    if a.size % 4:
        raise ValueError(f"{path}: not a whole number of 4-tuples")
    return a.reshape(-1, 4)


def write_block4(path: str, block4) -> None:
    write_array(path, np.asarray(block4).reshape(-1), np.int32)


def list_graphs(graph_dir: str):
    """Graph names in a directory, found the way the reference finds them: by <name>.config."""
    return sorted(f[: -len(".config")] for f in os.listdir(graph_dir) if f.endswith(".config"))


def read_sorted_graph(graph_dir: str, name: str):
    return (read_array(os.path.join(graph_dir, name + ".new_indptr")),
            read_array(os.path.join(graph_dir, name + ".new_indices")))


def write_graph(graph_dir: str, name: str, new_indptr, new_indices, orig_indptr=None, orig_indices=None) -> None:
    """Write a graph in the file set the reference harness opens (main.cu:62-65)."""
    os.makedirs(graph_dir, exist_ok=True)
    open(os.path.join(graph_dir, name + ".config"), "w").close()
    write_array(os.path.join(graph_dir, name + ".new_indptr"), new_indptr)
    write_array(os.path.join(graph_dir, name + ".new_indices"), new_indices)
    write_array(os.path.join(graph_dir, name + ".graph.ptrdump"), new_indptr if orig_indptr is None else orig_indptr)
    write_array(os.path.join(graph_dir, name + ".graph.edgedump"), new_indices if orig_indices is None else orig_indices)


def read_original_graph(graph_dir: str, name: str):
    """The CSR in its original node order (main.cu:64-65)."""
    return (read_array(os.path.join(graph_dir, name + ".graph.ptrdump")),
            read_array(os.path.join(graph_dir, name + ".graph.edgedump")))


def degree_sort_files(graph_dir: str, name: str, relabel_cols: bool = True):
    """<name>.graph.ptrdump / .edgedump  ->  <name>.new_indptr / .new_indices: the degree-ordered
    files the harness and the partitioner read (main.cu:62-63, block_level_partition.py:31-32).
    The reference ships its graphs already ordered and has no code for this step; here it is one
    call of the library's degree sort (rows ascending by degree, ties by original id, column ids
    renamed by the same permutation unless relabel_cols is False).  The permutation is written
    beside them as <name>.perm (perm[new_row] = original row) so that results can be put back in
    the original order.  Returns (perm, new_indptr, new_indices)."""
    from . import degree_sort
    indptr, indices = read_original_graph(graph_dir, name)
    perm, new_indptr, new_indices, _ = degree_sort.degree_sort(indptr, indices, None, relabel_cols=relabel_cols)
    write_array(os.path.join(graph_dir, name + ".new_indptr"), new_indptr)
    write_array(os.path.join(graph_dir, name + ".new_indices"), new_indices)
    write_array(os.path.join(graph_dir, name + ".perm"), perm)
    return perm, new_indptr, new_indices


if __name__ == "__main__":
    import sys
    if len(sys.argv) != 3:
        sys.exit("usage: python -m accelgcn.graphio <graph_dir> <name>    (degree-sorts <name>.graph.ptrdump/.edgedump)")
    _perm, _ip, _ix = degree_sort_files(sys.argv[1], sys.argv[2])
    print(f"{sys.argv[2]}: {len(_ip) - 1} rows, {len(_ix)} nonzeros -> .new_indptr / .new_indices / .perm")
