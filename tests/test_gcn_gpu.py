"""The dense transform (tcgen05 TF32 GEMM) and the two-layer GCN forward against fp64 numpy.

TF32 keeps 10 mantissa bits of each operand: with K = 128 products per output the tolerance is
rel 2e-3 of the row scale (sum_k |h_k w_kn|) -- stated here, separate from the fp32 SpMM gate."""
import numpy as np
import pytest

from conftest import require_cuda

pytestmark = pytest.mark.gpu


def _check_gemm(h, w, z):
    ref = h.astype(np.float64) @ w.astype(np.float64)
    scale = np.abs(h).astype(np.float64) @ np.abs(w).astype(np.float64)
    err = np.abs(z - ref)
    assert not np.isnan(z).any()
    assert np.all(err <= 2e-3 * scale + 1e-6), f"max err/scale {np.max(err / (scale + 1e-30)):.2e}"


@pytest.mark.parametrize("m", [1, 127, 128, 129, 1000, 128 * 148 + 5, 300_000])
def test_gemm_tf32_matches_fp64(m):
    import torch
    from accelgcn import gemm, synth
    dev = require_cuda()
    h = synth.features(m, 128, 11 + m, dev)
    w = synth.glorot(128, 128, 5, 8, dev)
    z = torch.full((m, 128), float("nan"), device=dev)
    gemm.gemm_tf32(h, w, out=z)
    torch.cuda.synchronize()
    _check_gemm(h.cpu().numpy(), w.cpu().numpy(), z.cpu().numpy())


def test_gemm_identity_and_strided_rows():
    import torch
    from accelgcn import gemm, synth
    dev = require_cuda()
    # values exactly representable in TF32 times the identity: the product is exact
    h = torch.randint(-512, 512, (5000, 128), device=dev).to(torch.float32) / 64.0
    z = gemm.gemm_tf32(h, torch.eye(128, device=dev))
    assert torch.equal(z, h)
    # operands with a row stride larger than 128; columns outside the product are untouched
    big = synth.features(777, 256, 3, dev)
    out = torch.full((777, 192), float("nan"), device=dev)
    w = synth.glorot(128, 128, 5, 9, dev)
    gemm.gemm_tf32(big[:, 64:192], w, out=out[:, :128])
    torch.cuda.synchronize()
    _check_gemm(big[:, 64:192].cpu().numpy(), w.cpu().numpy(), out[:, :128].cpu().numpy())
    assert torch.isnan(out[:, 128:]).all()


def test_gemm_rejects_other_shapes():
    import torch
    from accelgcn import gemm, AccelGcnError
    dev = require_cuda()
    with pytest.raises(AccelGcnError, match="K = N = 128"):
        gemm.gemm_tf32(torch.zeros((10, 64), device=dev), torch.zeros((64, 128), device=dev))


def test_spmm_fused_relu():
    import torch
    from accelgcn import synth, degree_sort, partition, spmm
    from oracle import oracle
    dev = require_cuda()
    g = synth.make_config(4, dev, 0.02)
    _, ip, ix, v = degree_sort.degree_sort_device(g.indptr, g.indices, g.vals)
    b4 = partition.block_level_partition_device(ip)
    x = synth.features(g.n, 64, 4, dev)
    plan = spmm.SpmmPlan(b4, ix, g.n, g.n)
    y = torch.full((g.n, 64), float("nan"), device=dev)
    plan.run(ix, v, x, y, relu=True)
    torch.cuda.synchronize()
    plan.close()
    ref = np.maximum(oracle.spmm_csr(ip.cpu().numpy(), ix.cpu().numpy(), v.cpu().numpy(), x.cpu().numpy()), 0)
    y = y.cpu().numpy()
    assert (y >= 0).all() and np.all(np.abs(y - ref) <= 1e-4 * np.abs(ref) + 5e-4)


@pytest.mark.parametrize("world", [1, 3])
def test_two_layer_gcn_forward_matches_fp64(world):
    # config 5 scaled to 25 000 nodes; with world > 1 every rank's shard is run in this process and
    # the all-gather is assembled by hand (the collective itself is covered by the gloo tests)
    import torch
    import scipy.sparse as sp
    from accelgcn import synth, degree_sort, sharded, gemm
    dev = require_cuda()
    g = synth.make_config(5, dev, 0.0005)
    _, ip, ix, v = degree_sort.degree_sort_device(g.indptr, g.indices, g.vals)
    n = g.n
    x = synth.features(n, 128, 1005, dev)
    w1, w2 = synth.glorot(128, 128, 1005, 8, dev), synth.glorot(128, 128, 1005, 9, dev)
    shards = [sharded.ShardedSpmm(ip, ix, v, r, world) for r in range(world)]

    def layer(h_full, w):
        zs = [gemm.gemm_tf32(h_full[sh.row_range[0]:sh.row_range[1]].contiguous(), w) for sh in shards]
        zg = torch.cat(zs)
        outs = []
        for sh in shards:
            y = torch.empty((sh.n_local, 128), device=dev)
            sh.plan.run(sh.indices, sh.vals, zg, y, dim=128, ldx=128, ldy=128, relu=True)
            outs.append(y)
        return torch.cat(outs)

    out = layer(layer(x, w1), w2).cpu().numpy()
    a = sp.csr_matrix((v.cpu().numpy().astype(np.float64), ix.cpu().numpy(), ip.cpu().numpy()), shape=(n, n))
    h1 = np.maximum(a @ (x.cpu().numpy().astype(np.float64) @ w1.cpu().numpy().astype(np.float64)), 0)
    ref = np.maximum(a @ (h1 @ w2.cpu().numpy().astype(np.float64)), 0)
    scale = np.abs(ref).max()
    assert np.all(np.abs(out - ref) <= 4e-3 * scale), np.abs(out - ref).max() / scale
    if world == 1:
        from accelgcn import gcn
        fwd = gcn.GcnForward(shards[0], [w1, w2])
        assert fwd.panel_cols is None
        assert torch.equal(fwd.forward(x).cpu(), torch.from_numpy(out))
        # the column-panelled schedule used across GPUs (exchange and multiply 32 columns at a time)
        paneled = gcn.GcnForward(shards[0], [w1, w2], panel_cols=32).forward(x).cpu().numpy()
        assert np.all(np.abs(paneled - ref) <= 4e-3 * scale)
        assert np.all(np.abs(paneled - out) <= 1e-5 + 1e-4 * np.abs(out))
    for sh in shards:
        sh.close()
