"""The CPU oracle of the SpMM kernel against scipy's CSR @ dense (no GPU)."""
import numpy as np
import pytest
import scipy.sparse as sp

from conftest import spmm_close, row_abs_scale
from oracle import oracle


def _random_sorted_csr(rng, n, heavy=()):
    deg = np.minimum((rng.pareto(1.2, n) * 2).astype(np.int64), n // 2)
    deg[rng.choice(n, len(heavy), replace=False)] = heavy
    deg = np.sort(deg)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    idx = np.concatenate([np.sort(rng.choice(n, d, replace=False)) for d in deg]).astype(np.int32)
    val = rng.uniform(0.05, 1.0, len(idx)).astype(np.float32)
    return indptr, idx, val


@pytest.mark.parametrize("dim", [16, 33, 60, 64, 100, 128])
def test_block4_kernel_model_matches_scipy(dim):
    rng = np.random.default_rng(dim)
    n = 1500
    indptr, idx, val = _random_sorted_csr(rng, n, heavy=(33, 385, 700, 1200))
    x = rng.uniform(-1, 1, (n, dim)).astype(np.float32)
    block4 = oracle.partition(indptr)
    y = oracle.spmm_block4(block4, idx, val, x, n)
    ref = sp.csr_matrix((val.astype(np.float64), idx, indptr), shape=(n, n)) @ x.astype(np.float64)
    assert spmm_close(y, ref, row_abs_scale(indptr, val, x)).all()
    assert spmm_close(oracle.spmm_csr(indptr, idx, val, x), ref).all()
    assert spmm_close(oracle.spmm_csr(indptr, idx, val, x, f32_accumulate=True), ref, row_abs_scale(indptr, val, x)).all()


def test_reference_kernel_semantics_on_prefilled_output():
    # Facts of spmm_accel.cu:82-99 the replacement has to know about: degree <= 32 rows are
    # stored, degree >= 33 rows are accumulated into what Y held, degree-0 rows are not written.
    rng = np.random.default_rng(1)
    deg = np.array([0, 0, 5, 32, 33, 400])
    n = 500
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    idx = np.concatenate([np.sort(rng.choice(n, d, replace=False)) for d in deg]).astype(np.int32)
    val = np.ones(len(idx), dtype=np.float32)
    x = rng.uniform(0, 1, (n, 16)).astype(np.float32)
    block4 = oracle.partition(indptr)
    y0 = np.full((len(deg), 16), 7.0, dtype=np.float32)
    clean = oracle.spmm_block4(block4, idx, val, x, len(deg))
    dirty = oracle.spmm_block4(block4, idx, val, x, len(deg), y0=y0)
    assert np.all(dirty[:2] == 7.0) and np.all(clean[:2] == 0.0)        # never written
    assert np.array_equal(dirty[2:4], clean[2:4])                        # stored
    assert np.allclose(dirty[4:], clean[4:] + 7.0, rtol=1e-5)            # accumulated


def test_out_of_range_index_is_reported():
    block4 = np.array([[1, 0, 0, (1 << 16) + 1]], dtype=np.int32)
    with pytest.raises(ValueError):
        oracle.spmm_block4(block4, np.array([5], np.int32), np.ones(1, np.float32), np.ones((3, 4), np.float32), 1)
