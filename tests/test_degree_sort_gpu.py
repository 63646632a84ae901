"""GPU degree sort + CSR permute against the CPU oracle (stable ascending argsort)."""
import numpy as np
import pytest

from conftest import require_cuda
from oracle import oracle

pytestmark = pytest.mark.gpu


def _check(g, relabel):
    from accelgcn import degree_sort
    ip, ix, v = g.indptr.numpy(), g.indices.numpy(), g.vals.numpy()
    got = degree_sort.degree_sort(ip, ix, v, relabel_cols=relabel)
    want = oracle.degree_sort(ip, ix, v, relabel_cols=relabel)
    for a, b, what in zip(got, want, ("perm", "indptr", "indices", "vals")):
        assert np.array_equal(a, b), what


@pytest.mark.parametrize("cfg,scale", [(1, 1.0), (2, 0.01), (3, 0.02), (4, 0.05), (5, 0.001)])
@pytest.mark.parametrize("relabel", [False, True])
def test_matches_oracle_on_synthetic_configs(cfg, scale, relabel):
    from accelgcn import synth
    require_cuda()
    _check(synth.make_config(cfg, "cpu", scale), relabel)


def test_device_entry_and_properties_at_scale():
    # 2 million rows, degrees up to 2^17 (three radix passes): oracle equality for the
    # permutation, then properties of the permuted matrix
    import torch
    from accelgcn import degree_sort
    dev = require_cuda()
    rng = np.random.default_rng(5)
    n = 2_000_000
    deg = np.minimum((rng.pareto(1.1, n) * 3).astype(np.int64), 130_000)
    deg[rng.integers(0, n, 3)] = [70_000, 131_000, 66_000]
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    assert indptr[-1] < 2**31
    nnz = int(indptr[-1])
    idx = rng.integers(0, n, nnz, dtype=np.int32)
    val = rng.random(nnz, dtype=np.float32)
    t_ip = torch.from_numpy(indptr.astype(np.int32)).to(dev)
    perm, nip, nix, nv = degree_sort.degree_sort_device(t_ip, torch.from_numpy(idx).to(dev),
                                                        torch.from_numpy(val).to(dev), relabel_cols=True)
    perm, nip = perm.cpu().numpy(), nip.cpu().numpy()
    assert np.array_equal(perm, np.argsort(deg, kind="stable"))
    assert np.array_equal(np.diff(nip.astype(np.int64)), deg[perm])
    inv = np.empty(n, dtype=np.int64); inv[perm] = np.arange(n)
    nix, nv = nix.cpu().numpy(), nv.cpu().numpy()
    for r in rng.integers(0, n, 200).tolist() + [n - 1, n - 2, n - 3]:
        o = perm[r]
        assert np.array_equal(nix[nip[r]:nip[r + 1]], inv[idx[indptr[o]:indptr[o + 1]]])
        assert np.array_equal(nv[nip[r]:nip[r + 1]], val[indptr[o]:indptr[o + 1]])
    assert np.isclose(float(nv.astype(np.float64).sum()), float(val.astype(np.float64).sum()), rtol=1e-9)


def test_all_rows_empty_and_single_row():
    from accelgcn import degree_sort
    require_cuda()
    perm, nip, nix, _ = degree_sort.degree_sort(np.zeros(6, dtype=np.int32), np.zeros(0, dtype=np.int32))
    assert perm.tolist() == [0, 1, 2, 3, 4] and nip.tolist() == [0] * 6 and len(nix) == 0
    perm, nip, nix, _ = degree_sort.degree_sort(np.array([0, 3], dtype=np.int32), np.array([0, 0, 0], dtype=np.int32))
    assert perm.tolist() == [0] and nip.tolist() == [0, 3] and nix.tolist() == [0, 0, 0]


def test_bad_input_is_an_error_not_a_fault():
    from accelgcn import degree_sort, AccelGcnError
    require_cuda()
    with pytest.raises(AccelGcnError):
        degree_sort.degree_sort(np.array([0, 2, 1], dtype=np.int32), np.array([0, 1], dtype=np.int32))
    with pytest.raises(AccelGcnError):       # column 9 cannot be relabelled in a 2-row matrix
        degree_sort.degree_sort(np.array([0, 1, 2], dtype=np.int32), np.array([0, 9], dtype=np.int32), relabel_cols=True)


def test_values_given_but_not_wanted_and_wrong_nnz():
    # the C ABI allows d_vals != NULL with d_new_vals == NULL (the values are simply not permuted),
    # and rejects an nnz that is not the matrix's own count instead of reading past the arrays
    import ctypes
    import torch
    from accelgcn import _lib, synth
    dev = require_cuda()
    lib = _lib.load()
    g = synth.make_config(1, dev, 0.25)
    n, nnz = g.n, g.nnz
    perm = torch.empty(n, dtype=torch.int32, device=dev)
    nip = torch.empty(n + 1, dtype=torch.int32, device=dev)
    nix = torch.full((nnz,), -1, dtype=torch.int32, device=dev)
    rc = lib.agcn_degree_sort_device(g.indptr.data_ptr(), g.indices.data_ptr(), g.vals.data_ptr(), n, nnz, 1,
                                     perm.data_ptr(), nip.data_ptr(), nix.data_ptr(), None, None)
    assert rc == _lib.OK, lib.agcn_last_error()
    torch.cuda.synchronize()
    want = oracle.degree_sort(g.indptr.cpu().numpy(), g.indices.cpu().numpy(), None, True)
    assert np.array_equal(perm.cpu().numpy(), want[0]) and np.array_equal(nix.cpu().numpy(), want[2])
    for wrong in (nnz + 4096, nnz - 1):
        rc = lib.agcn_degree_sort_device(g.indptr.data_ptr(), g.indices.data_ptr(), None, n, wrong, 0,
                                         perm.data_ptr(), nip.data_ptr(), nix.data_ptr(), None, None)
        assert rc == _lib.ERR_INVALID and b"nnz" in lib.agcn_last_error()
    torch.cuda.synchronize()


def test_row_pointers_at_any_alignment():
    # the degree pass reads four row pointers per 16-byte load where the caller's array allows it and
    # one at a time where it does not: the same matrix through pointers at offsets 0..3 words
    import torch
    from accelgcn import degree_sort, synth
    dev = require_cuda()
    g = synth.make_config(1, "cpu", 0.5)
    want = oracle.degree_sort(g.indptr.numpy(), g.indices.numpy(), None, True)
    ix = g.indices.to(dev)
    for shift in range(4):
        buf = torch.zeros(g.n + 1 + shift, dtype=torch.int32, device=dev)
        buf[shift:] = g.indptr.to(dev)
        view = buf[shift:]
        assert view.data_ptr() % 16 == (4 * shift) % 16
        perm, nip, nix, _ = degree_sort.degree_sort_device(view, ix, None, relabel_cols=True)
        assert np.array_equal(perm.cpu().numpy(), want[0]), shift
        assert np.array_equal(nip.cpu().numpy(), want[1]) and np.array_equal(nix.cpu().numpy(), want[2]), shift
