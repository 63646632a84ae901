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


def test_gemm_async_entry_and_status_word():
    import torch
    from accelgcn import gemm, synth
    dev = require_cuda()
    h = synth.features(70_000, 128, 3, dev)
    w = synth.glorot(128, 128, 5, 8, dev)
    z = torch.full((70_000, 128), float("nan"), device=dev)
    status = torch.full((1,), 77, dtype=torch.int32, device=dev)         # the call zeroes it on the stream
    gemm.gemm_tf32_async(h, w, z, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    _check_gemm(h.cpu().numpy(), w.cpu().numpy(), z.cpu().numpy())
    assert torch.equal(z, gemm.gemm_tf32(h, w))                          # same kernel, same bits


def test_gemm_bounded_wait_runs_out_and_the_next_call_succeeds():
    # failure detection without a fault: the self-test entry starves one pipeline wait (a load that
    # is never issued) under a spin limit of well under a millisecond; the kernel must leave through
    # its abort path -- status AGCN_ERR_CUDA, tensor memory freed -- and the device must stay usable
    import torch
    from accelgcn import gemm, synth, _lib
    dev = require_cuda()
    h = synth.features(40_000, 128, 4, dev)
    w = synth.glorot(128, 128, 5, 9, dev)
    z = torch.zeros((40_000, 128), device=dev)
    rc = gemm.selftest_timeout(h, w, z)
    assert rc == _lib.ERR_CUDA and b"ran out" in _lib.load().agcn_last_error()
    torch.cuda.synchronize()                                             # no sticky error: the context is intact
    for _ in range(2):
        z2 = gemm.gemm_tf32(h, w)
        torch.cuda.synchronize()
        _check_gemm(h.cpu().numpy(), w.cpu().numpy(), z2.cpu().numpy())


def _forward_reference(ip_h, ix_h, v_h, x_h, w1_h, w2_h):
    """CPU forward: fp32 storage, dense transform in fp64 row blocks, SpMM with fp64 accumulation (oracle)."""
    from oracle import oracle
    oracle.use_all_host_threads()

    def dense(h, w):
        out = np.empty((h.shape[0], w.shape[1]), dtype=np.float32)
        w64 = w.astype(np.float64)
        for a in range(0, h.shape[0], 1 << 18):
            out[a:a + (1 << 18)] = h[a:a + (1 << 18)].astype(np.float64) @ w64
        return out

    h1 = np.maximum(oracle.spmm_csr(ip_h, ix_h, v_h, dense(x_h, w1_h)), 0)
    return np.maximum(oracle.spmm_csr(ip_h, ix_h, v_h, dense(h1, w2_h)), 0)


@pytest.mark.parametrize("world,slices", [(1, 1), (3, 1), (4, 2)])
def test_two_layer_gcn_forward_matches_fp64(world, slices):
    # config 5 scaled to 25 000 nodes; with world > 1 every rank's block runs in this process
    # (contexts without a communicator) and the all-gather is assembled by hand; the NCCL exchange
    # itself runs in the multi-GPU benchmark and its layout is covered by the gloo tests
    import torch
    from accelgcn import synth, degree_sort, sharded, gemm, gcn
    dev = require_cuda()
    g = synth.make_config(5, dev, 0.0005)
    _, ip, ix, v = degree_sort.degree_sort_device(g.indptr, g.indices, g.vals)
    n = g.n
    x = synth.features(n, 128, 1005, dev)
    w1, w2 = synth.glorot(128, 128, 1005, 8, dev), synth.glorot(128, 128, 1005, 9, dev)
    shards = [sharded.ShardedSpmm(ip, ix, v, r, world, exchange_slices=slices, communicator=False) for r in range(world)]

    def layer(h_blocks, w):
        zs = [gemm.gemm_tf32(hb, w) for hb in h_blocks]
        zg = shards[0].assemble_gathered(zs)
        outs = []
        for sh in shards:
            y = torch.empty((sh.rows_per_block, 128), device=dev)
            sh.multiply_gathered(zg, y, relu=True)
            outs.append(y)
        return outs

    out_blocks = layer(layer([sh.to_block(x) for sh in shards], w1), w2)
    out = shards[0].from_blocks(out_blocks).cpu().numpy()
    ref = _forward_reference(ip.cpu().numpy(), ix.cpu().numpy(), v.cpu().numpy(), x.cpu().numpy(), w1.cpu().numpy(), w2.cpu().numpy())
    scale = np.abs(ref).max()
    assert np.all(np.abs(out - ref) <= 4e-3 * scale), np.abs(out - ref).max() / scale
    if world == 1:
        # the native forward (agcn_gcn2_forward_*) enqueues the same kernels: same bits
        fwd = gcn.GcnForward(shards[0], [w1, w2])
        got = fwd.forward(shards[0].to_block(x))
        torch.cuda.synchronize()
        times = fwd.status(timings=True)
        assert len(times) == 2 and all(t >= 0 for layer_t in times for t in layer_t)
        assert torch.equal(got, out_blocks[0])
        fwd.close()
    for sh in shards:
        sh.close()


def test_two_layer_gcn_forward_at_five_million_nodes():
    # configuration 5 at a tenth of its size (N = 5 000 000, ~1.07e8 nonzeros, 128 features): the whole
    # native forward against the CPU forward.  Tolerance: TF32 keeps 10 mantissa bits per operand of
    # the dense transform, so 4e-3 of the output scale (the SpMM itself is fp32 within 1e-4).
    import torch
    from accelgcn import synth, degree_sort, sharded, gcn
    dev = require_cuda()
    g = synth.make_config(5, dev, 0.1)
    _, ip, ix, v = degree_sort.degree_sort_device(g.indptr, g.indices, g.vals)
    n = g.n
    del g
    x = synth.features(n, 128, 1005, dev)
    w1, w2 = synth.glorot(128, 128, 1005, 8, dev), synth.glorot(128, 128, 1005, 9, dev)
    sh = sharded.ShardedSpmm(ip, ix, v, 0, 1)
    fwd = gcn.GcnForward(sh, [w1, w2])
    out_block = fwd.forward(sh.to_block(x))
    torch.cuda.synchronize()
    fwd.status()
    out = sh.from_blocks([out_block]).cpu().numpy()
    fwd.close(); sh.close()
    ref = _forward_reference(ip.cpu().numpy(), ix.cpu().numpy(), v.cpu().numpy(), x.cpu().numpy(), w1.cpu().numpy(), w2.cpu().numpy())
    scale = float(np.abs(ref).max())
    err = np.abs(out - ref)
    assert err.max() <= 4e-3 * scale, err.max() / scale
    # and tighter where it matters: the typical element, not just the worst one
    assert float(np.sqrt((err.astype(np.float64) ** 2).mean())) <= 4e-4 * scale


@pytest.mark.parametrize("m,n_cols", [(1, 64), (127, 500), (1000, 5000), (128 * 300 + 17, 40_000)])
def test_fused_layer_matches_fp64(m, n_cols):
    # Z2 = relu(A Z1) W for rows of 0..32 nonzeros: the sparse part in fp32 (rel 1e-4), the dense part in
    # TF32 (2e-3 of the row scale sum_k |h_k w_kn|)
    import torch
    from accelgcn import gemm, synth
    dev = require_cuda()
    rng = np.random.default_rng(m)
    deg = rng.integers(0, 33, m)
    deg[rng.integers(0, m, max(1, m // 50))] = 0
    deg[rng.integers(0, m, max(1, m // 50))] = 32
    ip = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    ix = rng.integers(0, n_cols, int(ip[-1])).astype(np.int32)
    v = rng.uniform(-1, 1, int(ip[-1])).astype(np.float32)
    z1 = synth.features(n_cols, 128, 77 + m, dev)
    w = synth.glorot(128, 128, 5, 9, dev)
    out = torch.full((m + 3, 128), float("nan"), device=dev)
    gemm.gcn_fused_layer(torch.from_numpy(ip).to(dev), torch.from_numpy(ix).to(dev), torch.from_numpy(v).to(dev), z1, w, m,
                         out=out[:m])
    torch.cuda.synchronize()
    assert torch.isnan(out[m:]).all()                       # rows past m_rows are not written
    z1_h, w_h = z1.cpu().numpy().astype(np.float64), w.cpu().numpy().astype(np.float64)
    h = np.zeros((m, 128))
    rows = np.repeat(np.arange(m), deg)
    np.add.at(h, rows, v[:, None].astype(np.float64) * z1_h[ix])
    h = np.maximum(h, 0)
    ref = h @ w_h
    scale = np.abs(h) @ np.abs(w_h)
    got = out[:m].cpu().numpy()
    assert not np.isnan(got).any()
    assert np.all(np.abs(got - ref) <= 2e-3 * scale + 1e-5), float(np.max(np.abs(got - ref) / (scale + 1e-30)))


def test_forward_with_fused_layer_boundary(monkeypatch):
    # AGCN_GCN_FUSED=1: the light rows of the block take the fused kernel between the layers, the others
    # SpMM + GEMM; the result must agree with the plain forward (same arithmetic, another summation order)
    import torch
    from accelgcn import synth, degree_sort, sharded, gcn
    dev = require_cuda()
    g = synth.make_config(5, dev, 0.002)
    _, ip, ix, v = degree_sort.degree_sort_device(g.indptr, g.indices, g.vals)
    x = synth.features(g.n, 128, 1005, dev)
    w1, w2 = synth.glorot(128, 128, 1005, 8, dev), synth.glorot(128, 128, 1005, 9, dev)
    sh = sharded.ShardedSpmm(ip, ix, v, 0, 1)
    xb = sh.to_block(x)
    plain = gcn.GcnForward(sh, [w1, w2])
    want = plain.forward(xb).clone()
    torch.cuda.synchronize()
    plain.status()
    plain.close()
    monkeypatch.setenv("AGCN_GCN_FUSED", "1")
    fused = gcn.GcnForward(sh, [w1, w2])
    got = fused.forward(xb)
    torch.cuda.synchronize()
    fused.status()
    deg = (ip[1:] - ip[:-1])
    assert int((deg <= 32).sum()) >= 128 * 64              # the fused path is really taken at this size
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) <= 2e-3 * scale
    fused.close(); sh.close()


def test_fused_layer_reports_a_column_out_of_range():
    import torch
    from accelgcn import gemm, synth, AccelGcnError
    dev = require_cuda()
    ip = torch.tensor([0, 2, 3], dtype=torch.int32, device=dev)
    ix = torch.tensor([1, 50, 7], dtype=torch.int32, device=dev)          # 50 is outside the 50 rows of Z1
    v = torch.ones(3, device=dev)
    z1 = synth.features(50, 128, 3, dev)
    w = torch.eye(128, device=dev)
    with pytest.raises(AccelGcnError, match="status 4"):
        gemm.gcn_fused_layer(ip, ix, v, z1, w, 2)
    ix[1] = 49
    got = gemm.gcn_fused_layer(ip, ix, v, z1, w, 2)                        # the device is fine: the next call succeeds
    want = torch.relu(torch.stack([z1[1] + z1[49], z1[7]]))
    assert torch.allclose(got, want, rtol=2e-3, atol=2e-3)
