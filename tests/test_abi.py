"""The C-ABI library loads without a GPU and exports exactly what include/accelgcn.h declares."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT, PKG

import importlib.util


def _build():
    spec = importlib.util.spec_from_file_location("agcn_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "accelgcn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(agcn_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_loads_and_exports_every_declared_symbol():
    path = _build()
    lib = ctypes.CDLL(path)
    declared = _declared_symbols()
    assert len(declared) >= 12
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in accelgcn.h but not exported"


def test_python_prototypes_cover_the_header():
    from accelgcn import _lib
    assert sorted(_lib.PROTOTYPES) == _declared_symbols()
    _build()
    lib = _lib.load()
    assert lib.agcn_version() >= 100
    assert lib.agcn_last_error() == b""


def test_argument_errors_need_no_gpu():
    # argument validation happens before any CUDA call
    from accelgcn import _lib
    _build()
    lib = _lib.load()
    n = ctypes.c_int64(0)
    assert lib.agcn_partition_device(None, 5, None, 0, ctypes.byref(n), None) == _lib.ERR_INVALID
    assert b"null" in lib.agcn_last_error()
    ip = np.zeros(1, dtype=np.int32)
    assert lib.agcn_partition_host(ip.ctypes.data, 0, None, 0, ctypes.byref(n)) == _lib.ERR_INVALID
    assert b"empty graph" in lib.agcn_last_error()
    assert lib.agcn_spmm_run(None, None, None, None, 0, None, 0, 4, None) == _lib.ERR_INVALID


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from accelgcn import _lib
    monkeypatch.setenv("ACCELGCN_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    with pytest.raises(FileNotFoundError):
        _lib.load()


def test_host_partition_raises_on_empty_graph_like_the_script():
    from accelgcn import partition
    with pytest.raises(IndexError):
        partition.block_level_partition(np.array([0], dtype=np.int32))


def test_graphio_roundtrip(tmp_path):
    from accelgcn import graphio
    b = np.arange(24, dtype=np.int32).reshape(-1, 4)
    graphio.write_block4(str(tmp_path / "g.block4"), b)
    assert np.array_equal(graphio.read_block4(str(tmp_path / "g.block4")), b)
    graphio.write_graph(str(tmp_path / "graphs"), "g", [0, 1, 3], [1, 0, 1])
    assert graphio.list_graphs(str(tmp_path / "graphs")) == ["g"]
    ip, ix = graphio.read_sorted_graph(str(tmp_path / "graphs"), "g")
    assert ip.tolist() == [0, 1, 3] and ix.tolist() == [1, 0, 1]
    (tmp_path / "bad.block4").write_bytes(b"\0" * 20)
    with pytest.raises(ValueError):
        graphio.read_block4(str(tmp_path / "bad.block4"))


def test_synthetic_graphs_are_seeded_and_well_formed():
    from accelgcn import synth
    a = synth.make_config(1, "cpu", 0.25)
    b = synth.make_config(1, "cpu", 0.25)
    assert np.array_equal(a.indices.numpy(), b.indices.numpy()) and np.array_equal(a.vals.numpy(), b.vals.numpy())
    ip, ix = a.indptr.numpy().astype(np.int64), a.indices.numpy()
    assert ip[0] == 0 and ip[-1] == len(ix) and np.all(np.diff(ip) >= 1)      # self loops: no empty row
    assert abs(a.nnz / (a.n * 8.0) - 1) < 0.25
    for r in (0, 17, a.n - 1):
        row = ix[ip[r]:ip[r + 1]]
        assert np.all(np.diff(row) > 0) and r in row                       # sorted, unique, self loop
    # symmetric pattern and GCN normalisation
    import scipy.sparse as sp
    m = sp.csr_matrix((a.vals.numpy(), ix, ip), shape=(a.n, a.n))
    assert (abs(m - m.T) > 1e-7).nnz == 0
    d = np.diff(ip).astype(np.float64)
    r = 123
    assert np.allclose(m[r].toarray().ravel()[ix[ip[r]:ip[r + 1]]], 1 / np.sqrt(d[r] * d[ix[ip[r]:ip[r + 1]]]), rtol=1e-6)
    g4 = synth.make_config(4, "cpu", 0.01)
    assert g4.vals.min() > 0 and g4.vals.max() <= 1 and g4.info["max_degree"] > 384
    x = synth.features(100, 60, 1001, "cpu")
    assert x.shape == (100, 60) and x.min() >= -1 and x.max() < 1
