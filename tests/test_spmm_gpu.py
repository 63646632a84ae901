"""Parity of the GPU SpMM with the oracle (CSR x dense in fp64, and the thread-for-thread fp32
restatement of the reference kernel), through the C ABI.  Tolerance: rel 1e-4 / abs 1e-5."""
import os

import numpy as np
import pytest

from conftest import require_cuda, spmm_close, row_abs_scale
from oracle import oracle

pytestmark = pytest.mark.gpu


class Case:
    """A degree-ordered synthetic graph on host and device with its .block4 metadata."""

    def __init__(self, cfg, scale, sort=True, empty_rows=()):
        import torch
        from accelgcn import synth, degree_sort, partition
        self.dev = require_cuda()
        g = synth.make_config(cfg, "cpu", scale)
        ip, ix, v = g.indptr.numpy(), g.indices.numpy(), g.vals.numpy()
        if len(empty_rows):                       # drop every nonzero of the named rows
            deg = np.diff(ip.astype(np.int64))
            keep = np.ones(len(ix), dtype=bool)
            for r in empty_rows:
                keep[ip[r]:ip[r + 1]] = False
                deg[r] = 0
            ix, v = ix[keep], v[keep]
            ip = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
        if sort:
            _, ip, ix, v = degree_sort.degree_sort(ip, ix, v, relabel_cols=True)
        self.n, self.indptr, self.idx, self.val = g.n, ip, ix, v
        self.block4 = partition.block_level_partition(ip)
        self.seed = g.info["seed"]
        self.t = {k: torch.from_numpy(a).to(self.dev) for k, a in
                  (("block4", self.block4), ("idx", ix), ("val", v))}

    def x(self, dim):
        from accelgcn import synth
        return synth.features(self.n, dim, self.seed, "cpu").numpy()

    def run(self, x, prefill=float("nan")):
        import torch
        from accelgcn import spmm
        xt = torch.from_numpy(x).to(self.dev)
        y = torch.full((self.n, x.shape[1]), prefill, dtype=torch.float32, device=self.dev)
        spmm.spmm(self.t["block4"], self.t["idx"], self.t["val"], xt, self.n, out=y)
        return y.cpu().numpy()

    def check(self, x, y):
        ref = oracle.spmm_csr(self.indptr, self.idx, self.val, x)
        ok = spmm_close(y, ref, row_abs_scale(self.indptr, self.val, x))
        assert not np.isnan(y).any(), "some of Y was not written"
        assert ok.all(), f"{(~ok).sum()} elements out of tolerance, first at {np.argwhere(~ok)[0]}"


@pytest.fixture(scope="module")
def cfg1():
    return Case(1, 1.0)


@pytest.fixture(scope="module")
def cfg4_small():
    return Case(4, 0.04)      # 20 000 rows, one row of 8 000 nonzeros: heavy rows crossing units


@pytest.mark.parametrize("dim", list(range(16, 129, 4)) + [1, 7, 17, 33, 61, 99, 127])
def test_config1_every_dim_against_oracle(cfg1, dim):
    x = cfg1.x(dim)
    cfg1.check(x, cfg1.run(x))


@pytest.mark.parametrize("dim", [16, 32, 60, 64, 100, 128, 45])
def test_skewed_graph_heavy_rows(cfg4_small, dim):
    x = cfg4_small.x(dim)
    y = cfg4_small.run(x)
    cfg4_small.check(x, y)


def test_matches_reference_kernel_restatement_in_fp32(cfg1):
    # against the thread-for-thread fp32 model of spmm_accel.cu on a zeroed Y
    x = cfg1.x(60)
    y = cfg1.run(x)
    ref32 = oracle.spmm_block4(cfg1.block4, cfg1.idx, cfg1.val, x, cfg1.n)
    assert spmm_close(y, ref32, row_abs_scale(cfg1.indptr, cfg1.val, x)).all()


@pytest.mark.parametrize("cfg,scale,dim", [(2, 0.02, 64), (3, 0.02, 64), (5, 0.002, 128)])
def test_other_configs_scaled_down(cfg, scale, dim):
    c = Case(cfg, scale)
    x = c.x(dim)
    c.check(x, c.run(x))


def test_overwrites_output_and_is_bitwise_reproducible(cfg4_small):
    x = cfg4_small.x(64)
    a = cfg4_small.run(x, prefill=float("nan"))
    b = cfg4_small.run(x, prefill=123.0)
    c = cfg4_small.run(x, prefill=-1e30)
    assert np.array_equal(a, b) and np.array_equal(a, c)


def test_unsorted_rows_and_zero_degree_rows_anywhere():
    # .block4 of an unsorted graph (zero-degree rows in the middle and at the end)
    n = 12_000
    c = Case(3, 0.005, sort=False, empty_rows=(0, 1, 2, 77, 78, 5000, n - 2, n - 1))
    assert c.n == n and (np.diff(c.indptr) == 0).sum() >= 8 and (np.diff(np.diff(c.indptr)) < 0).any()
    for dim in (32, 60, 9):
        x = c.x(dim)
        c.check(x, c.run(x))


def test_wide_and_strided_operands(cfg1):
    import torch
    from accelgcn import spmm
    dev = cfg1.dev
    # dim > 128 is processed in 128-column panels; ld > dim exercises the row strides
    x = cfg1.x(200)
    cfg1.check(x, cfg1.run(x))
    xw = torch.from_numpy(cfg1.x(96)).to(dev)
    ybuf = torch.full((cfg1.n, 128), float("nan"), dtype=torch.float32, device=dev)
    plan = spmm.SpmmPlan(cfg1.t["block4"], cfg1.t["idx"], cfg1.n, cfg1.n)
    plan.run(cfg1.t["idx"], cfg1.t["val"], xw[:, :64], ybuf[:, 32:96], dim=64, ldx=96, ldy=128)
    torch.cuda.synchronize()
    plan.close()
    out = ybuf.cpu().numpy()
    cfg1.check(xw[:, :64].cpu().numpy().copy(), out[:, 32:96].copy())
    assert np.isnan(out[:, :32]).all() and np.isnan(out[:, 96:]).all()       # nothing outside the panel touched


def test_linearity_at_full_size_config3_shape():
    # property that needs no oracle at a size the CPU cannot check quickly: A(ax + by) = aAx + bAy
    import torch
    from accelgcn import synth, degree_sort, partition, spmm
    dev = require_cuda()
    g = synth.make_config(3, dev, 0.25)          # 600 000 rows, ~15 M nonzeros
    _, ip, ix, v = degree_sort.degree_sort_device(g.indptr, g.indices, g.vals, relabel_cols=True)
    b4 = partition.block_level_partition_device(ip)
    x1 = synth.features(g.n, 64, 1, dev)
    x2 = synth.features(g.n, 64, 2, dev)
    y1 = spmm.spmm(b4, ix, v, x1, g.n)
    y2 = spmm.spmm(b4, ix, v, x2, g.n)
    y3 = spmm.spmm(b4, ix, v, 0.5 * x1 - 2.0 * x2, g.n)
    assert torch.allclose(y3, 0.5 * y1 - 2.0 * y2, rtol=1e-4, atol=1e-5)
    # and a sampled-row check against the fp64 CSR product
    rows = torch.randint(0, g.n, (300,), device=dev).tolist() + [g.n - 1]
    ip_h, ix_h, v_h, x_h = ip.cpu().numpy(), ix.cpu().numpy(), v.cpu().numpy(), x1.cpu().numpy().astype(np.float64)
    y_h = y1.cpu().numpy()
    for r in rows:
        s = slice(ip_h[r], ip_h[r + 1])
        ref = (v_h[s].astype(np.float64)[:, None] * x_h[ix_h[s]]).sum(0)
        assert np.all(np.abs(y_h[r] - ref) <= 1e-5 + 1e-4 * np.abs(ref)), r


def test_host_buffer_entry_point(cfg1):
    from accelgcn import spmm
    h = spmm.HostSpmm()
    for dim in (60, 128):
        x = cfg1.x(dim)
        y = h(cfg1.block4, cfg1.idx, cfg1.val, x, cfg1.n)
        cfg1.check(x, y)
    # constructor / run split of the plug-in: the graph goes up once, every run moves X and Y only
    h.set_graph(cfg1.block4, cfg1.idx, cfg1.val, cfg1.n, cfg1.n)
    for dim in (16, 100):
        x = cfg1.x(dim)
        cfg1.check(x, h.run(x))
    h.close()
    h2 = spmm.HostSpmm()
    with pytest.raises(spmm._lib.AccelGcnError, match="no graph set"):
        h2._n_rows, h2._n_cols = cfg1.n, cfg1.n
        h2.run(cfg1.x(16))
    h2.close()


def test_plugin_class_mirrors_reference_do_test(cfg1, tmp_path):
    # SPMM_ACCEL usage as in main.cu:131,146,166: buffers of dim_max columns, .block4 read from
    # ../block_level_meta/<graph>.block4 on every do_test, vin/vout re-read per dim
    import torch
    from accelgcn import spmm, graphio
    os.makedirs(tmp_path / "block_level_meta")
    graphio.write_block4(str(tmp_path / "block_level_meta" / "g.block4"), cfg1.block4)
    dev, n, dim_max = cfg1.dev, cfg1.n, 128
    vin = torch.from_numpy(cfg1.x(dim_max)).to(dev).reshape(-1)
    vout = torch.zeros(n * dim_max, dtype=torch.float32, device=dev)
    accel = spmm.SpmmAccel("g", torch.from_numpy(cfg1.indptr).to(dev), cfg1.t["idx"], cfg1.t["val"], vin, vout,
                           n, len(cfg1.idx), dim_max, meta_dir=str(tmp_path / "block_level_meta"))
    for dim in (60, 128):
        assert accel.do_test(False, dim) == 0.0
        x = vin[: n * dim].reshape(n, dim).cpu().numpy()
        cfg1.check(x, vout[: n * dim].reshape(n, dim).cpu().numpy())
    assert accel.do_test(True, 64) > 0.0


def test_invalid_input_is_rejected_not_faulted(cfg1):
    import torch
    from accelgcn import spmm, AccelGcnError
    dev = cfg1.dev
    bad_idx = cfg1.t["idx"].clone()
    bad_idx[5] = cfg1.n + 3
    with pytest.raises(AccelGcnError, match="column index"):
        spmm.SpmmPlan(cfg1.t["block4"], bad_idx, cfg1.n, cfg1.n)
    bad_b4 = cfg1.t["block4"].clone()
    bad_b4[3, 2] = len(cfg1.idx)                      # loc_begin past the end
    with pytest.raises(AccelGcnError, match="nonzero range"):
        spmm.SpmmPlan(bad_b4, cfg1.t["idx"], cfg1.n, cfg1.n)
    bad_b4 = cfg1.t["block4"].clone()
    bad_b4[0, 1] = cfg1.n                             # row out of range
    with pytest.raises(AccelGcnError, match="rows"):
        spmm.SpmmPlan(bad_b4, cfg1.t["idx"], cfg1.n, cfg1.n)
    torch.cuda.synchronize()


@pytest.mark.skipif(not oracle.ref_available(), reason="oracle/_ref not built (needs the reference tree at build time)")
@pytest.mark.parametrize("dim", [16, 60, 64, 100, 128])
def test_parity_with_the_reference_kernel_itself(cfg1, dim):
    # the reference's spmm_kernel_accel, compiled from its own sources for sm_100a, on a zeroed Y
    x = cfg1.x(dim)
    ref = oracle.ref_accel_spmm(cfg1.block4, cfg1.indptr, cfg1.idx, cfg1.val, x)
    y = cfg1.run(x)
    assert spmm_close(y, ref, row_abs_scale(cfg1.indptr, cfg1.val, x)).all()
    # the C restatement of that kernel is pinned by the same run
    model = oracle.spmm_block4(cfg1.block4, cfg1.idx, cfg1.val, x, cfg1.n)
    assert spmm_close(model, ref, row_abs_scale(cfg1.indptr, cfg1.val, x)).all()


@pytest.mark.skipif(not oracle.ref_available(), reason="oracle/_ref not built")
def test_parity_with_the_reference_kernel_heavy_rows(cfg4_small):
    x = cfg4_small.x(64)
    ref = oracle.ref_accel_spmm(cfg4_small.block4, cfg4_small.indptr, cfg4_small.idx, cfg4_small.val, x)
    y = cfg4_small.run(x)
    assert spmm_close(y, ref, row_abs_scale(cfg4_small.indptr, cfg4_small.val, x)).all()
    cs = oracle.ref_cusparse_spmm(cfg4_small.indptr, cfg4_small.idx, cfg4_small.val, x)
    assert spmm_close(y, cs, row_abs_scale(cfg4_small.indptr, cfg4_small.val, x)).all()


@pytest.mark.parametrize("world,slices,ranges", [(2, 1, 1), (5, 1, 1), (4, 3, 1), (8, 2, 1), (4, 1, 3), (1, 1, 2)])
def test_row_sharded_product_on_one_gpu_equals_unsharded(cfg4_small, world, slices, ranges):
    # every rank's block built and multiplied in this one process (contexts without a communicator:
    # the all-gather is replaced by assembling the gathered operand by hand): two row ranges per
    # rank, column ids renamed to gathered positions, block-local .block4
    import torch
    from accelgcn import sharded
    c = cfg4_small
    dev = c.dev
    ip, ix, v = (torch.from_numpy(a).to(dev) for a in (c.indptr, c.idx, c.val))
    x = c.x(64)
    xt = torch.from_numpy(x).to(dev)
    # (ranges > 1: the block's columns tiled into equal ranges of the gathered operand, one exchange)
    shards = [sharded.ShardedSpmm(ip, ix, v, r, world, exchange_slices=slices, communicator=False, column_ranges=ranges)
              for r in range(world)]
    gathered = shards[0].assemble_gathered([sh.to_block(xt) for sh in shards])
    blocks = []
    for sh in shards:
        y = torch.full((sh.rows_per_block, 64), float("nan"), dtype=torch.float32, device=dev)
        sh.multiply_gathered(gathered, y)
        blocks.append(y)
    torch.cuda.synchronize()
    y = shards[0].from_blocks(blocks).cpu().numpy()
    c.check(x, y)
    for sh, blk in zip(shards, blocks):                        # padding rows multiply to zero
        assert torch.all(blk[sh.rows_of() < 0] == 0)
    # the device layout is the host layout (agcn_balanced_blocks), and it balances rows and nonzeros
    ranges, per = sharded.balanced_blocks(c.indptr, world)
    per = -(-per // slices) * slices
    for r, sh in enumerate(shards):
        assert sh.rows_per_block == per and np.array_equal(sh.rows_of().cpu().numpy(), sharded.block_rows(ranges, per, r))
    nnz = np.array([sh.local_nnz for sh in shards])
    assert nnz.sum() == len(c.idx) and nnz.max() - nnz.min() <= 2 * np.diff(c.indptr).max()
    for sh in shards:
        sh.close()


def test_cpp_harness_same_cli_and_output_as_the_reference(cfg1, tmp_path):
    # spmm_test <graph> <dim>, run from a build directory beside graphs/ and block_level_meta/
    # (README.md:70-73): checks against cuSPARSE, then prints the reference's timing lines
    import subprocess, importlib.util
    from conftest import PKG
    from accelgcn import graphio
    spec = importlib.util.spec_from_file_location("agcn_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec); spec.loader.exec_module(mod)
    exe = mod.build_harness()
    graphio.write_graph(str(tmp_path / "graphs"), "synth1", cfg1.indptr, cfg1.idx)
    os.makedirs(tmp_path / "block_level_meta"); os.makedirs(tmp_path / "build")
    graphio.write_block4(str(tmp_path / "block_level_meta" / "synth1.block4"), cfg1.block4)
    out = subprocess.run([exe, "synth1", "60"], cwd=tmp_path / "build", capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "validation pass!" in out.stdout and "validation fail!" not in out.stdout
    lines = [l.split() for l in out.stdout.splitlines() if l.startswith("0/0 synth1 60 ")]
    assert [l[3] for l in lines] == ["cusparse", "accel", "accel_event"] and all(float(l[4]) > 0 for l in lines)


def test_graph_without_nonzeros_gives_zeros():
    # no tuples at all: every row is zero-filled, nothing else is launched
    import torch
    from accelgcn import spmm
    dev = require_cuda()
    n = 1000
    b4 = torch.zeros((0, 4), dtype=torch.int32, device=dev)
    empty_i = torch.zeros(0, dtype=torch.int32, device=dev)
    empty_v = torch.zeros(0, dtype=torch.float32, device=dev)
    for dim in (64, 7):
        x = torch.ones((n, dim), device=dev)
        y = torch.full((n, dim), float("nan"), device=dev)
        spmm.spmm(b4, empty_i, empty_v, x, n, out=y)
        assert torch.equal(y, torch.zeros_like(y))


def test_single_heavy_row_spanning_many_units():
    # one row of 50 000 nonzeros = 131 tuples = 17 units: all of it goes through the carry path
    import torch
    from accelgcn import partition, spmm
    dev = require_cuda()
    rng = np.random.default_rng(8)
    n, d = 60_000, 50_000
    indptr = np.array([0, d], dtype=np.int32)
    idx = np.sort(rng.choice(n, d, replace=False)).astype(np.int32)
    val = rng.uniform(0, 1, d).astype(np.float32)
    x = rng.uniform(-1, 1, (n, 100)).astype(np.float32)
    b4 = partition.block_level_partition(indptr)
    assert len(b4) == 131
    y = spmm.spmm(torch.from_numpy(b4).to(dev), torch.from_numpy(idx).to(dev), torch.from_numpy(val).to(dev),
                  torch.from_numpy(x).to(dev), 1).cpu().numpy()
    ref = oracle.spmm_csr(indptr, idx, val, x)
    assert spmm_close(y, ref, row_abs_scale(indptr, val, x)).all()


def test_full_size_config2_checksum_and_sampled_rows():
    # the headline workload at its full size (250 000 nodes, ~1.2e8 nonzeros): properties that need
    # no full oracle -- 1^T (A X) = (1^T A) X in fp64, a row sample against the fp64 product, and
    # bit-identical output from two runs
    import torch
    from accelgcn import synth, degree_sort, partition, spmm
    dev = require_cuda()
    g = synth.make_config(2, dev, 1.0)
    _, ip, ix, v = degree_sort.degree_sort_device(g.indptr, g.indices, g.vals, relabel_cols=True)
    b4 = partition.block_level_partition_device(ip)
    n, dim = g.n, 64
    x = synth.features(n, dim, 1002, dev)
    plan = spmm.SpmmPlan(b4, ix, n, n)
    y1 = torch.full((n, dim), float("nan"), device=dev)
    y2 = torch.full((n, dim), 7.0, device=dev)
    plan.run(ix, v, x, y1)
    plan.run(ix, v, x, y2)
    torch.cuda.synchronize()
    plan.close()
    assert torch.equal(y1, y2)
    col_weight = torch.zeros(n, dtype=torch.float64, device=dev).index_add_(0, ix.to(torch.int64), v.to(torch.float64))
    want = col_weight @ x.to(torch.float64)                      # (1^T A) X
    got = y1.to(torch.float64).sum(0)
    assert torch.allclose(got, want, rtol=1e-6, atol=1e-6 * float(col_weight.abs().sum())), (got - want).abs().max()
    ip_h = ip.cpu().numpy()
    rows = np.unique(np.concatenate([np.random.default_rng(0).integers(0, n, 200), [0, n - 1, n - 2]]))
    for r in rows:
        a, b = int(ip_h[r]), int(ip_h[r + 1])
        ref = (v[a:b].to(torch.float64)[:, None] * x[ix[a:b].to(torch.int64)].to(torch.float64)).sum(0)
        err = (y1[r].to(torch.float64) - ref).abs()
        assert bool((err <= 1e-5 + 1e-4 * ref.abs()).all()), int(r)


# ----------------------------------------------------------------------------------------
# the configurations at the sizes the benchmark numbers are quoted on
# ----------------------------------------------------------------------------------------
def _full_config_on_device(cfg):
    import torch
    from accelgcn import synth, degree_sort, partition
    dev = require_cuda()
    g = synth.make_config(cfg, dev, 1.0)
    _, ip, ix, v = degree_sort.degree_sort_device(g.indptr, g.indices, g.vals, relabel_cols=True)
    b4 = partition.block_level_partition_device(ip)
    seed = g.info["seed"]
    n = g.n
    del g
    torch.cuda.empty_cache()
    return dev, n, seed, ip, ix, v, b4


def _checksum_and_rows(n, ip, ix, v, x, y, n_sample=200):
    """1^T (A X) = (1^T A) X in fp64, and a row sample (with the lightest and the heaviest rows)
    against the fp64 product, at the parity tolerance rel 1e-4 / abs 1e-5 scaled by the row's
    absolute sum."""
    import torch
    dev = x.device
    assert not torch.isnan(y).any()
    col_weight = torch.zeros(n, dtype=torch.float64, device=dev).index_add_(0, ix.to(torch.int64), v.to(torch.float64))
    want = col_weight @ x.to(torch.float64)
    got = y.to(torch.float64).sum(0)
    assert torch.allclose(got, want, rtol=1e-6, atol=1e-6 * float(col_weight.abs().sum())), float((got - want).abs().max())
    ip_h = ip.cpu().numpy()
    rows = np.unique(np.concatenate([np.random.default_rng(0).integers(0, n, n_sample), [0, 1, n - 3, n - 2, n - 1]]))
    xmax = float(x.abs().max())
    for r in rows:
        a, b = int(ip_h[r]), int(ip_h[r + 1])
        ref = (v[a:b].to(torch.float64)[:, None] * x[ix[a:b].to(torch.int64)].to(torch.float64)).sum(0)
        scale = max(1.0, float(v[a:b].abs().sum()) * xmax)
        err = (y[r].to(torch.float64) - ref).abs()
        assert bool((err <= 1e-5 * scale + 1e-4 * ref.abs()).all()), (int(r), float(err.max()))


@pytest.fixture(scope="module")
def cfg2_full():
    return _full_config_on_device(2)


@pytest.mark.parametrize("dim", [32, 128])
def test_full_size_config2_other_widths(cfg2_full, dim):
    # dim 128 is the launch the benchmark's roofline is quoted on, and the only one where the
    # two 64-column passes are chosen automatically (X = 128 MB against a 126 MB L2)
    import torch
    from accelgcn import synth, spmm
    dev, n, seed, ip, ix, v, b4 = cfg2_full
    x = synth.features(n, dim, seed, dev)
    plan = spmm.SpmmPlan(b4, ix, n, n)
    y = torch.full((n, dim), float("nan"), device=dev)
    plan.run(ix, v, x, y)
    torch.cuda.synchronize()
    launches = plan.info()["launches_last_run"]
    plan.close()
    if dim == 128:
        assert launches >= 2            # two column passes (plus the carry kernels if any row crosses units)
    _checksum_and_rows(n, ip, ix, v, x, y)


def test_full_size_config2_column_tiled(cfg2_full):
    # the column-tiled product at dim 128 (3 ranges): same checks, and within the parity tolerance of
    # the un-tiled product element by element (only the order of the fp32 additions differs)
    import torch
    from accelgcn import synth, spmm, _lib
    dev, n, seed, ip, ix, v, b4 = cfg2_full
    x = synth.features(n, 128, seed, dev)
    k = _lib.load().agcn_spmm_tiled_suggest(n, n, int(ix.numel()), 128)
    assert 2 <= k <= 8
    tiled = spmm.TiledSpmmPlan(ip, ix, v, n, n, dim=128)
    assert tiled.info()["n_ranges"] == k and sum(tiled.info()["range_nnz"]) == int(ix.numel())
    y1 = torch.full((n, 128), float("nan"), device=dev)
    y2 = torch.full((n, 128), 3.0, device=dev)
    tiled.run(x, y1)
    tiled.run(x, y2)
    torch.cuda.synchronize()
    tiled.close()
    assert torch.equal(y1, y2)                               # bit-identical from run to run
    _checksum_and_rows(n, ip, ix, v, x, y1)
    plan = spmm.SpmmPlan(b4, ix, n, n)
    y0 = torch.empty((n, 128), device=dev)
    plan.run(ix, v, x, y0)
    torch.cuda.synchronize()
    plan.close()
    assert bool(((y1 - y0).abs() <= 1e-5 + 1e-4 * y0.abs()).all())


@pytest.mark.parametrize("panel", [32, 64])
def test_forced_column_passes_on_small_graphs(cfg1, cfg4_small, panel, monkeypatch):
    # AGCN_SPMM_PANEL (read at plan creation) forces the pass loop -- and the reuse of the carry
    # scratch between passes -- on inputs small enough for the full oracle
    monkeypatch.setenv("AGCN_SPMM_PANEL", str(panel))
    for case in (cfg1, cfg4_small):
        for dim in (128, 100, 61):
            x = case.x(dim)
            case.check(x, case.run(x))


def test_full_size_config3():
    # N = 2 400 000, ~6e7 nonzeros, dim 64: the whole product against the CPU oracle (fp64 accumulation)
    import torch
    from accelgcn import synth, spmm
    dev, n, seed, ip, ix, v, b4 = _full_config_on_device(3)
    x = synth.features(n, 64, seed, dev)
    y = torch.full((n, 64), float("nan"), device=dev)
    spmm.spmm(b4, ix, v, x, n, out=y)
    oracle.use_all_host_threads()
    ip_h, ix_h, v_h, x_h = ip.cpu().numpy(), ix.cpu().numpy(), v.cpu().numpy(), x.cpu().numpy()
    ref = oracle.spmm_csr(ip_h, ix_h, v_h, x_h)
    ok = spmm_close(y.cpu().numpy(), ref, row_abs_scale(ip_h, v_h, x_h))
    assert ok.all(), f"{(~ok).sum()} elements out of tolerance, first at {np.argwhere(~ok)[0]}"


@pytest.fixture(scope="module")
def cfg4_full():
    dev, n, seed, ip, ix, v, b4 = _full_config_on_device(4)
    host = {k: t.cpu().numpy() for k, t in (("ip", ip), ("ix", ix), ("v", v), ("b4", b4))}
    return dev, n, seed, ip, ix, v, b4, host


@pytest.mark.parametrize("dim", list(range(16, 129, 4)))
def test_full_size_config4_sweep(cfg4_full, dim):
    # N = 500 000, max degree ~9e4, every width of the configuration: against the CPU oracle and
    # (where it was built) against the reference's own kernel on the same arrays
    import torch
    from accelgcn import synth, spmm
    dev, n, seed, ip, ix, v, b4, h = cfg4_full
    x = synth.features(n, dim, seed, dev)
    y = torch.full((n, dim), float("nan"), device=dev)
    spmm.spmm(b4, ix, v, x, n, out=y)
    y_h, x_h = y.cpu().numpy(), x.cpu().numpy()
    oracle.use_all_host_threads()
    scale = row_abs_scale(h["ip"], h["v"], x_h)
    ok = spmm_close(y_h, oracle.spmm_csr(h["ip"], h["ix"], h["v"], x_h), scale)
    assert ok.all(), f"{(~ok).sum()} elements out of tolerance, first at {np.argwhere(~ok)[0]}"
    if oracle.ref_available() and dim % 16 == 0:
        ref = oracle.ref_accel_spmm(h["b4"], h["ip"], h["ix"], h["v"], x_h)
        assert spmm_close(y_h, ref, scale).all()


@pytest.mark.parametrize("dim", [17, 61, 99, 127])
def test_unaligned_widths_padded_copy_equals_scalar_path(cfg4_small, dim, monkeypatch):
    # dims that are not multiples of 4: the default copies X into aligned rows and runs the 16-byte
    # path; AGCN_SPMM_PAD=0 keeps the 4-byte gathers.  Both against the oracle, and equal to each other
    # within the tolerance (the order of additions inside a row differs between the two).
    x = cfg4_small.x(dim)
    y_pad = cfg4_small.run(x)
    cfg4_small.check(x, y_pad)
    monkeypatch.setenv("AGCN_SPMM_PAD", "0")
    y_scalar = cfg4_small.run(x)
    cfg4_small.check(x, y_scalar)
    assert spmm_close(y_pad, y_scalar, row_abs_scale(cfg4_small.indptr, cfg4_small.val, x)).all()


@pytest.mark.parametrize("case_name", ["cfg1", "cfg4_small"])
def test_column_tiled_small(case_name, request):
    # tiled plan with several range layouts (one of them empty), ReLU, an unaligned width and the
    # range-by-range entry, against the oracle
    import torch
    from accelgcn import spmm
    c = request.getfixturevalue(case_name)
    dev = c.dev
    ip = torch.from_numpy(c.indptr).to(dev)
    n = c.n
    for bounds in ([0, n], [0, n // 2, n], [0, n // 3, n // 3, n - 5, n]):
        tiled = spmm.TiledSpmmPlan(ip, c.t["idx"], c.t["val"], n, n, bounds=bounds)
        for dim, relu in ((64, False), (128, True), (33, True)):
            x = c.x(dim)
            xt = torch.from_numpy(x).to(dev)
            y = torch.full((n, dim), float("nan"), device=dev)
            tiled.run(xt, y, relu=relu)
            y2 = torch.full((n, dim), float("nan"), device=dev)
            for k in range(len(bounds) - 1):
                tiled.run(xt, y2, relu=relu, only_range=k)
            torch.cuda.synchronize()
            assert torch.equal(y, y2)
            ref = oracle.spmm_csr(c.indptr, c.idx, c.val, x)
            if relu:
                ref = np.maximum(ref, 0)
            assert spmm_close(y.cpu().numpy(), ref, row_abs_scale(c.indptr, c.val, x)).all(), (bounds, dim)
        tiled.close()


def test_host_batch_and_streamed_graph(cfg1, cfg4_small):
    # the pipelined host-buffer calls: several products on a resident graph, and graph + products in
    # one call (A uploaded and multiplied range by range); bit-identical to the one-product call
    import torch
    from accelgcn import spmm
    for c in (cfg1, cfg4_small):
        h = spmm.HostSpmm()
        dims = [32, 64, 128, 60, 33]
        xs = [np.ascontiguousarray(c.x(d)) for d in dims]
        ys = h.step_batch(c.block4, c.idx, c.val, xs[:4], c.n)              # streamed (all widths multiples of 4)
        for x, y in zip(xs[:4], ys):
            c.check(x, y)
        t = h.last_timing()                                                  # where the time of that call went
        assert 0 <= t["first_kernel_started"] <= t["last_kernel_finished"] <= t["last_y_downloaded"] + 1e-3
        assert t["a_uploaded"] > 0 and t["host_all_enqueued"] >= t["host_plan_built"] > 0
        ys_all = h.step_batch(c.block4, c.idx, c.val, xs, c.n)              # 33 columns: upload first, then multiply
        for x, y in zip(xs, ys_all):
            c.check(x, y)
        h.set_graph(c.block4, c.idx, c.val, c.n, c.n)
        ys_res = h.run_batch(xs)
        for a, b in zip(ys_all, ys_res):
            assert np.array_equal(a, b)
        for x, y in zip(xs, ys_res):
            assert np.array_equal(h.run(x), y)
        for a, b in zip(ys, ys_res[:4]):
            assert np.array_equal(a, b)
        # pinned buffers take the same path
        px = [torch.from_numpy(x).pin_memory() for x in xs[:3]]
        py = [torch.empty((c.n, d), dtype=torch.float32).pin_memory() for d in dims[:3]]
        h.run_batch(px, outs=py)
        for y, ref in zip(py, ys_res[:3]):
            assert np.array_equal(y.numpy(), ref)
        # a column id out of range is rejected (by the check that runs ahead of each range), nothing faults
        bad = c.idx.copy()
        bad[len(bad) // 2] = c.n + 7
        with pytest.raises(spmm._lib.AccelGcnError, match="column index"):
            h.step_batch(c.block4, bad, c.val, xs[:3], c.n)
        ys_again = h.step_batch(c.block4, c.idx, c.val, xs[:3], c.n)        # and the context is still good
        for a, b in zip(ys_again, ys_res[:3]):
            assert np.array_equal(a, b)
        h.close()


def test_streamed_graph_in_several_ranges_and_malformed_block4():
    # a graph large enough (2.4e7 nonzeros) for the streamed call to cut A into several upload ranges:
    # bit-identical to the resident product; and tuples that would put a cut outside the arrays or out of
    # order (the cuts are taken from the caller's .block4 before the plan has validated it) are an error,
    # not a fault
    from accelgcn import spmm
    c = Case(2, 0.2)
    assert len(c.idx) * 8 >> 25 >= 4
    h = spmm.HostSpmm()
    xs = [np.ascontiguousarray(c.x(d)) for d in (32, 64)]
    ys = h.step_batch(c.block4, c.idx, c.val, xs, c.n)
    for x, y in zip(xs, ys):
        assert np.array_equal(y, c.run(x))
    n_units = (len(c.block4) + 7) // 8
    for unit, loc in ((n_units // 3, len(c.idx) + 5), (n_units // 2, 3), (2 * n_units // 3, -7)):
        bad = c.block4.copy()
        bad[unit * 8, 2] = loc
        with pytest.raises(spmm._lib.AccelGcnError):
            h.step_batch(bad, c.idx, c.val, xs, c.n)
    bad = c.block4.copy()
    bad[(n_units // 2) * 8, 1] = c.n + 1                 # row of a unit's first tuple past the matrix
    with pytest.raises(spmm._lib.AccelGcnError):
        h.step_batch(bad, c.idx, c.val, xs, c.n)
    ys_again = h.step_batch(c.block4, c.idx, c.val, xs, c.n)           # the context is still good
    for a, b in zip(ys_again, ys):
        assert np.array_equal(a, b)
    h.close()


def test_cpp_harness_full_sweep_mode(cfg1, tmp_path):
    # spmm_test with no arguments: every graph of ../graphs at every dim 16..128 step 1
    # (main.cu:195-219), here on two small graphs; with checking forced on, every product validates
    import subprocess, importlib.util
    from conftest import PKG
    from accelgcn import graphio, degree_sort, partition, synth
    spec = importlib.util.spec_from_file_location("agcn_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec); spec.loader.exec_module(mod)
    exe = mod.build_harness()
    os.makedirs(tmp_path / "block_level_meta"); os.makedirs(tmp_path / "build")
    graphio.write_graph(str(tmp_path / "graphs"), "synth1", cfg1.indptr, cfg1.idx)
    graphio.write_block4(str(tmp_path / "block_level_meta" / "synth1.block4"), cfg1.block4)
    g = synth.make_config(4, "cpu", 0.004)
    _, ip, ix, _ = degree_sort.degree_sort(g.indptr.numpy(), g.indices.numpy(), None)
    graphio.write_graph(str(tmp_path / "graphs"), "synth4", ip, ix)
    graphio.write_block4(str(tmp_path / "block_level_meta" / "synth4.block4"), partition.block_level_partition(ip))
    env = dict(os.environ, AGCN_TEST_CHECK_ALL="1")
    out = subprocess.run([exe], cwd=tmp_path / "build", capture_output=True, text=True, timeout=1200, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "validation fail!" not in out.stdout
    accel = [l.split() for l in out.stdout.splitlines() if " accel " in l]
    assert len(accel) == 2 * 113 and {l[1] for l in accel} == {"synth1", "synth4"}
    assert sorted({int(l[2]) for l in accel}) == list(range(16, 129))
    assert out.stdout.count("validation pass!") == 2 * 113


def test_degree_sort_files_front_end(tmp_path):
    # original-order files -> .new_indptr / .new_indices / .perm, as one library call
    from accelgcn import graphio, synth
    g = synth.make_config(1, "cpu", 0.25)
    ip, ix = g.indptr.numpy(), g.indices.numpy()
    d = str(tmp_path / "graphs")
    graphio.write_graph(d, "g", np.zeros(1, np.int32), np.zeros(0, np.int32), orig_indptr=ip, orig_indices=ix)
    perm, nip, nix = graphio.degree_sort_files(d, "g")
    want = oracle.degree_sort(ip, ix, None, True)
    assert np.array_equal(perm, want[0]) and np.array_equal(nip, want[1]) and np.array_equal(nix, want[2])
    rip, rix = graphio.read_sorted_graph(d, "g")
    assert np.array_equal(rip, nip) and np.array_equal(rix, nix)
    assert np.array_equal(graphio.read_array(os.path.join(d, "g.perm")), perm)


def test_gather_probe_runs():
    import ctypes
    from accelgcn import _lib
    require_cuda()
    gbs = ctypes.c_double(0.0)
    _lib.check(_lib.load().agcn_probe_gather_bandwidth(1 << 16, 64, 1 << 22, 3, 5, ctypes.byref(gbs)))
    assert gbs.value > 100.0            # GB/s: any working GPU is far above this
