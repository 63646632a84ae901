"""Benchmark of the Accel-GCN SpMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2]

One step = one pass of the SpMM over the workload's dense widths (config 2: dim 32, 64 and
128 on the 250 000-node / ~1.2e8-nonzero heavy graph).  Prints ONE JSON line.

  value     whole-job GFLOP/s (2 * nnz * dim per product) with everything resident in HBM
  e2e       the same through the host-buffer C-ABI call: .block4, indices, values and X go up
            from pinned host memory and Y comes back, every step, inside the timed region
  roofline  compulsory HBM bytes of the widest product / its CUDA-event time, against the
            measured copy bandwidth of this pool's B200s
  cpu_baseline  the CPU restatement of the reference path (oracle) on a bounded row sample, with the
            Python partition walk and scipy's single-threaded csr @ dense beside it

`--impl reference` times that CPU path alone, with all host threads, on the same workload.
Under torchrun with N > 1 the matrix is row-sharded (two row ranges per rank: equal rows and equal
nonzeros) and every step all-gathers the dense operand over NCCL inside the library (strong
scaling: the total work is fixed).
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "iccad-accel-gcn_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np   # noqa: E402

WORKLOADS = {
    # name: (config id, scale, dims)
    "cfg2": (2, 1.0, (32, 64, 128)),
    "cfg1": (1, 1.0, (60,)),
    "cfg3": (3, 1.0, (64,)),
    "cfg4": (4, 1.0, tuple(range(16, 129, 4))),
    "cfg2-small": (2, 0.04, (32, 64, 128)),      # for quick checks of the script itself
    # two-layer GCN forward relu(A relu(A X W1) W2), 128 features (step = one forward)
    "cfg5": (5, 1.0, (128,)),
    "cfg5-5m": (5, 0.1, (128,)),
    "cfg5-1m": (5, 0.02, (128,)),
    "cfg5-small": (5, 0.002, (128,)),
}
GCN_WORKLOADS = ("cfg5", "cfg5-5m", "cfg5-1m", "cfg5-small")
# "replicas": the 16 graphs of the reference's benchmark set whose .block4 files it ships, rebuilt
# from the degree sequence each file inverts to (tests/golden/block4_kat.json) with seeded uniform
# random column ids -- the real edge lists are a download that is not available offline
WORKLOADS["replicas"] = (0, 1.0, (64,))
METRIC, UNIT = "spmm_gflops", "GFLOP/s"
FALLBACK_HBM_GBS = 6650.0
# (workload, dim, kernel variant) -> dram__bytes_read + dram__bytes_write per product, from the ncu captures
# summarised under profiles/ (same command as the default run)
NCU_TRAFFIC_BYTES = {("cfg2", 128, "column-tiled"): 1.770e9, ("cfg2", 128, "two 64-column passes"): 3.971e9,
                     ("cfg3", 64, "one pass"): 9.524e9}


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy read+write)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (earlier measurement on this pool)"


def min_bytes(nnz, n_blocks, n_rows, n_cols, dim):
    """Compulsory HBM traffic of one product: A once, .block4 once, X once, Y once."""
    return 8 * nnz + 16 * n_blocks + 4 * dim * n_cols + 4 * dim * n_rows


def workload_description(name, g_info, n, nnz, n_blocks, dims):
    return {"workload": f"{name}: synthetic config {g_info['config']} graph, N={n}, nnz={nnz}, "
                        f"max degree {g_info['max_degree']}, {n_blocks} .block4 tuples, "
                        f"SpMM at dim {'/'.join(map(str, dims))} per step",
            "dims": list(dims), "n": n, "nnz": nnz, "n_blocks": n_blocks,
            "l2": "no flush: A (8 B per nonzero) is larger than L2 and is streamed by every product"}


# ----------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU while a region runs."""
    FIELDS = ("uuid,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str):
        self.uuid = uuid
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        rows = [[c.strip() for c in line.split(",")] for line in self.file if line.count(",") >= 7]
        self.file.close()
        os.unlink(self.file.name)
        mine = [r for r in rows if self.uuid and self.uuid in r[0]] or rows
        sm, mx, pw, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in mine:
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); pw.append(float(r[3]))
            except ValueError:
                continue
            for nme, flag in zip(names, r[4:8]):
                if flag == "Active":
                    reasons.add(nme)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------
def build_workload(name, dev):
    """Synthetic graph -> degree sort -> (sorted CSR on `dev`, generator info).  On a CUDA device
    the ordering is done by the library; on the CPU (reference arm without a GPU) by the oracle."""
    import torch
    from accelgcn import synth
    cfg, scale, dims = WORKLOADS[name]
    g = synth.make_config(cfg, dev, scale)
    if torch.device(dev).type == "cuda":
        from accelgcn import degree_sort, partition
        degree_sort.degree_sort_device(g.indptr[:1025].clone() - g.indptr[0], g.indices[:int(g.indptr[1024])], None, relabel_cols=False)  # warm-up
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        _perm, ip, ix, v = degree_sort.degree_sort_device(g.indptr, g.indices, g.vals, relabel_cols=True)
        t1 = time.perf_counter()
        b4 = partition.block_level_partition_device(ip)
        t2 = time.perf_counter()
        # one-shot wall-clock times of the preprocessing calls (they include their scratch allocation)
        g.info["preprocess_ms"] = {"degree_sort_and_csr_permute": (t1 - t0) * 1e3, "block_level_partition": (t2 - t1) * 1e3,
                                   "n_blocks": int(b4.shape[0])}
        del b4
    else:
        from oracle import oracle
        _perm, ip, ix, v = oracle.degree_sort(g.indptr.numpy(), g.indices.numpy(), g.vals.numpy(), True)
        ip, ix, v = torch.from_numpy(ip), torch.from_numpy(ix), torch.from_numpy(v)
    return g, ip, ix, v, dims


def build_workload_reference(name):
    """The same degree-ordered matrix for the reference arm, without loading this repository's
    library: the generator is torch arithmetic (run on the GPU when there is one, only to save
    minutes of CPU sorting) and the ordering is the oracle's (numpy)."""
    import torch
    from accelgcn import synth
    from oracle import oracle
    cfg, scale, dims = WORKLOADS[name]
    g = synth.make_config(cfg, "cuda:0" if torch.cuda.is_available() else "cpu", scale)
    ip_h, ix_h, v_h = g.indptr.cpu().numpy(), g.indices.cpu().numpy(), g.vals.cpu().numpy()
    info = dict(g.info)
    n = g.n
    del g
    _perm, ip_h, ix_h, v_h = oracle.degree_sort(ip_h, ix_h, v_h, True)
    return n, info, ip_h, ix_h, v_h, dims


def row_sample(ip_h, ix_h, v_h, stride):
    """Every stride-th row of a host CSR matrix (degree-ordered, so a strided sample keeps the degree mix)."""
    if stride <= 1:
        return ip_h, ix_h, v_h
    rows = np.arange(0, len(ip_h) - 1, stride)
    deg = (ip_h[rows + 1] - ip_h[rows]).astype(np.int64)
    sp = np.concatenate([[0], np.cumsum(deg)])
    src = np.repeat(ip_h[rows].astype(np.int64) - sp[:-1], deg) + np.arange(sp[-1])
    return sp.astype(np.int32), ix_h[src], v_h[src]


def cpu_spmm_rate(ip_h, ix_h, v_h, xs, budget_s):
    """Times the CPU restatement (oracle, fp32, all OpenMP threads) on a strided row sample sized to
    take about budget_s seconds over all widths.  Returns (GFLOP/s, seconds, sample description, stride)."""
    from oracle import oracle
    oracle.use_all_host_threads()
    n, nnz = len(ip_h) - 1, len(ix_h)
    dsum = sum(x.shape[1] for x in xs)
    probe_stride = max(1, n // 2048)
    sp, si, sv = row_sample(ip_h, ix_h, v_h, probe_stride)
    oracle.spmm_csr(sp, si, sv, xs[0], f32_accumulate=True)                  # warm the threads
    t0 = time.perf_counter()
    for x in xs:
        oracle.spmm_csr(sp, si, sv, x, f32_accumulate=True)
    rate = 2.0 * len(si) * dsum / max(time.perf_counter() - t0, 1e-6)        # flop/s on the probe
    want_nnz = rate * budget_s / (2.0 * dsum)
    stride = max(1, int(np.ceil(nnz / max(want_nnz, 1.0))))
    sp, si, sv = row_sample(ip_h, ix_h, v_h, stride)
    t0 = time.perf_counter()
    for x in xs:
        oracle.spmm_csr(sp, si, sv, x, f32_accumulate=True)
    dt = time.perf_counter() - t0
    desc = (f"every {stride}th row of the degree-ordered matrix ({len(sp) - 1} rows, {len(si)} nonzeros), "
            f"all widths, full X")
    return 2.0 * len(si) * dsum / dt / 1e9, dt, desc, stride


def cpu_reference_extras(ip_h, ix_h, v_h, xs, stride, budget_s=6.0):
    """What the reference itself runs on the CPU for this path, timed on bounded samples: the
    partition walk of block_level_partition.py:48-103 (pure Python, one core -- the restatement in
    oracle.partition_py; the script itself does not travel to the GPU box) and scipy's csr @ dense
    in fp32 (single-threaded), the product its results are checked against."""
    import scipy.sparse as sp
    from oracle import oracle
    n = len(ip_h) - 1
    rows = min(n, 400_000)
    t0 = time.perf_counter()
    b4 = oracle.partition_py(np.concatenate([[0], np.cumsum(np.diff(ip_h[: rows + 1].astype(np.int64)))]))
    dt_part = time.perf_counter() - t0
    sp_ip, sp_ix, sp_v = row_sample(ip_h, ix_h, v_h, max(stride, 1))
    # scipy is ~50x slower than the threaded port: shrink the sample to stay within the budget
    keep = max(1, int(len(sp_ip) - 1))
    a = sp.csr_matrix((sp_v, sp_ix, sp_ip), shape=(keep, xs[0].shape[0]))
    probe_rows = max(1, keep // 64)
    t0 = time.perf_counter()
    a[:probe_rows] @ xs[0]
    est = (time.perf_counter() - t0) * 64 * sum(x.shape[1] for x in xs) / xs[0].shape[1]
    frac = min(1.0, budget_s / max(est, 1e-6))
    a = a[: max(1, int(keep * frac))]
    t0 = time.perf_counter()
    for x in xs:
        a @ x
    dt_sp = time.perf_counter() - t0
    return {"partition_walk": {"rows_per_s": rows / dt_part, "rows": rows, "tuples": int(len(b4)), "seconds": dt_part,
                               "cores": 1, "what": "pure-Python walk of block_level_partition.py:48-103 (oracle.partition_py) "
                                                   "on the first rows of the workload's row pointers"},
            "scipy_csr_dense": {"value": 2.0 * a.nnz * sum(x.shape[1] for x in xs) / dt_sp / 1e9, "unit": UNIT, "cores": 1,
                                "seconds": dt_sp, "sample": f"{a.shape[0]} rows / {a.nnz} nonzeros of the port's sample, all widths, fp32"}}


# ----------------------------------------------------------------------------------------
def reference_arm(args, rank, world):
    """The reference's CPU path for the SpMM (its only CPU code is the Python partitioner; the
    product it is checked against is CSR x dense), restated in C with OpenMP in oracle/.  Nothing
    of this repository's library is loaded in this arm."""
    if rank != 0:
        return
    from oracle import oracle
    from accelgcn import synth
    n, info, ip_h, ix_h, v_h, dims = build_workload_reference(args.workload)
    nnz = len(ix_h)
    n_blocks = int(len(oracle.partition(ip_h)))
    xs = [synth.features(n, d, info["seed"], "cpu").numpy() for d in dims]
    dsum = sum(dims)
    per_step = min(2.0, 150.0 / max(args.steps + args.warmup, 1))
    _rate, _dt, desc, stride = cpu_spmm_rate(ip_h, ix_h, v_h, xs, per_step)
    sp, si, sv = row_sample(ip_h, ix_h, v_h, stride)
    for _ in range(args.warmup):
        for x in xs:
            oracle.spmm_csr(sp, si, sv, x, f32_accumulate=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for x in xs:
            oracle.spmm_csr(sp, si, sv, x, f32_accumulate=True)
    dt = time.perf_counter() - t0
    gflops = 2.0 * len(si) * dsum * args.steps / dt / 1e9
    info = {"config": WORKLOADS[args.workload][0], "max_degree": int(np.diff(ip_h).max())}
    line = {"impl": "reference", "metric": METRIC, "value": gflops, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_description(args.workload, info, n, nnz, n_blocks, dims),
            "cpu_baseline": {"value": gflops, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
                             "sample": "each step: " + desc,
                             "reference_cpu_path": cpu_reference_extras(ip_h, ix_h, v_h, xs, stride)},
            "e2e": {"value": gflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------
def gather_peaks(dims):
    """Measured ceiling of the gather itself: GB/s of whole-row reads from an L2-resident table (32 MB)
    with the SpMM's access shape, per row width (agcn_probe_gather_bandwidth)."""
    import ctypes
    from accelgcn import _lib
    lib = _lib.load()
    out = {}
    for d in sorted(set(dims)):
        if d not in (32, 64, 128):
            continue
        rows = (32 << 20) // (4 * d)             # a 32 MB table: a power-of-two number of rows
        best = 0.0
        for resident in (5, 0):            # the SpMM's residency, and whatever the registers allow
            gbs = ctypes.c_double(0.0)
            _lib.check(lib.agcn_probe_gather_bandwidth(rows, d, (2 << 30) // (4 * d), 5, resident, ctypes.byref(gbs)))
            best = max(best, gbs.value)
        out[d] = best
    return out


def pcie_peaks(dev, mb=512):
    """Plain pinned-memory copies of `mb` MiB each way (torch, CUDA events): what this box's PCIe link
    delivers, the ceiling of the end-to-end numbers."""
    import torch
    h = torch.empty(mb << 20, dtype=torch.uint8).pin_memory()
    d = torch.empty(mb << 20, dtype=torch.uint8, device=dev)
    out = {}
    for name, (dst, src) in (("h2d_gbs", (d, h)), ("d2h_gbs", (h, d))):
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            dst.copy_(src, non_blocking=True)
        b.record()
        torch.cuda.synchronize(dev)
        out[name] = 3 * (mb << 20) / (a.elapsed_time(b) / 1e3) / 1e9
    return out


def checksum_check(ip, ix, v, n, xs_full, ys, shard_of, col_of, dims, dev, world):
    """1^T (A X) = (1^T A) X in fp64 over all ranks' rows (and column groups), and a row sample of this
    rank's block against the fp64 product from the whole matrix (every rank still holds it at this point)."""
    import torch
    import torch.distributed as dist
    col_weight = torch.zeros(n, dtype=torch.float64, device=dev).index_add_(0, ix.to(torch.int64), v.to(torch.float64))
    ok = True
    worst = 0.0
    for d in dims:
        rows = shard_of[d].rows_of()
        c0, c1 = col_of[d]
        valid = torch.nonzero(rows >= 0).reshape(-1)
        pick = valid[torch.randint(0, valid.numel(), (64,), device=dev)]
        pick = torch.unique(torch.cat([pick, valid[:1], valid[-1:]]))
        got = torch.zeros(d, dtype=torch.float64, device=dev)
        got[c0:c1] = ys[d].to(torch.float64).sum(0)
        if world > 1:
            dist.all_reduce(got)
        want = col_weight @ xs_full[d].to(torch.float64)
        ok = ok and bool(torch.allclose(got, want, rtol=1e-6, atol=1e-6 * float(col_weight.abs().sum())))
        for j in pick.tolist():
            r = int(rows[j])
            a, b = int(ip[r]), int(ip[r + 1])
            ref = (v[a:b].to(torch.float64)[:, None] * xs_full[d][ix[a:b].to(torch.int64), c0:c1].to(torch.float64)).sum(0)
            scale = max(1.0, float(v[a:b].abs().sum()))
            err = float(((ys[d][j].to(torch.float64) - ref).abs() - 1e-4 * ref.abs()).max())
            worst = max(worst, err / scale)
    flag = torch.tensor([1.0 if (ok and worst <= 1e-5) else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return {"ok": bool(flag.item() > 0), "what": "1^T(AX) = (1^T A)X in fp64 over all ranks, plus 66 sampled rows per rank and width "
                                                  "against the fp64 product (rel 1e-4 / abs 1e-5 x row scale)"}


def ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from accelgcn import synth, sharded, spmm as spmm_mod, _lib

    assert torch.cuda.is_available(), "bench.py needs a CUDA device: the library has no CPU fallback"
    _lib.load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()

    g, ip, ix, v, dims = build_workload(args.workload, dev)
    n, nnz = g.n, int(ix.numel())
    if world > 1:
        # the products of a step are independent, so their order is free: widest first.  Its exchange is the
        # one left exposed, and the narrow products -- the ones that live on X staying in L2 -- then run
        # after the last exchange has landed instead of under the incoming data of the wide ones.
        dims = tuple(sorted(dims, reverse=True))
    # one block of A per rank (two row ranges: equal rows and equal nonzeros); the dense operands and
    # results are block rows.  On one GPU the block is the whole matrix and nothing is exchanged.
    # (--slices S: widths of at least --slices-min-dim columns exchange their operand in S row slices and
    # multiply slice by slice, on a second context of the same layout; narrower widths keep one slice)
    sliced = world > 1 and args.slices > 1
    # rows x features (--feature-groups F): a product of at least --feature-groups-min-dim columns is
    # multiplied as F independent row-sharded products of dim / F columns, each over world / F ranks with its
    # own communicator -- 1 / F of the exchange among 1 / F of the ranks, blocks of F times the rows
    fg = 1
    if world > 1:
        fg = args.feature_groups if args.feature_groups > 0 else (4 if world % 8 == 0 else 2 if world % 2 == 0 else 1)
        assert world % fg == 0, "--feature-groups must divide the number of GPUs"
    fg_dims = [d for d in dims if fg > 1 and not sliced and d % fg == 0 and d >= args.feature_groups_min_dim
               and d // fg >= args.feature_groups_min_width]
    shard = sharded.ShardedSpmm(ip, ix, v, rank, world)
    shard_of = {d: shard for d in dims}
    col_of = {d: (0, d) for d in dims}
    ranges_of = {d: 1 for d in dims}
    lib = _lib.load()
    if sliced and any(d >= args.slices_min_dim for d in dims):
        shard_sliced = sharded.ShardedSpmm(ip, ix, v, rank, world, exchange_slices=args.slices)
        shard_of.update({d: shard_sliced for d in dims if d >= args.slices_min_dim})
    elif world > 1 and args.tiled != "off":
        # a gathered operand that does not fit L2 is multiplied column range by column range (as on one GPU):
        # widths that want the same number of ranges share one more context of the same layout
        by_ranges = {}
        for d in dims:
            k = lib.agcn_spmm_tiled_suggest(shard.rows_per_block, shard.n_gathered, shard.local_nnz, d)
            if k > 1 and d not in fg_dims:
                by_ranges.setdefault(k, []).append(d)
        for k, ds in by_ranges.items():
            tiled_shard = sharded.ShardedSpmm(ip, ix, v, rank, world, column_ranges=k)
            shard_of.update({d: tiled_shard for d in ds})
            ranges_of.update({d: "tiled" for d in ds})
    if fg_dims:
        row_rank, row_world, fgroup, _members = sharded.feature_groups(rank, world, fg)
        groups = [dist.new_group(ranks=list(range(j, world, fg))) for j in range(fg)]      # every rank makes every group
        grp = groups[fgroup] if row_world > 1 else None
        fg_shard = sharded.ShardedSpmm(ip, ix, v, row_rank, row_world, group=grp)
        fg_tiled = {}
        for d in fg_dims:
            w = d // fg
            col_of[d] = (fgroup * w, (fgroup + 1) * w)
            k = 1
            if args.tiled != "off":
                k = lib.agcn_spmm_tiled_suggest(fg_shard.rows_per_block, fg_shard.n_gathered, fg_shard.local_nnz, w)
            if k > 1 and k not in fg_tiled:
                fg_tiled[k] = sharded.ShardedSpmm(ip, ix, v, row_rank, row_world, group=grp, column_ranges=k)
            shard_of[d] = fg_tiled[k] if k > 1 else fg_shard
            ranges_of[d] = "tiled" if k > 1 else 1
    per = shard.rows_per_block
    n_blocks_local = int(shard.n_blocks)
    nb = torch.tensor([n_blocks_local], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(nb)
    n_blocks = int(nb.item())
    xs_full = {d: synth.features(n, d, g.info["seed"], dev) for d in dims}
    xs = {d: shard_of[d].to_block(xs_full[d] if col_of[d] == (0, d) else xs_full[d][:, col_of[d][0]:col_of[d][1]].contiguous())
          for d in dims}
    ys = {d: torch.empty_like(xs[d]) for d in dims}
    # single GPU: a product whose X does not stay in L2 runs column-tiled (A regrouped by column range)
    tiled = {}
    if world == 1 and args.tiled != "off":
        lib = _lib.load()
        for d in dims:
            k = lib.agcn_spmm_tiled_suggest(n, n, nnz, d)
            if k > 1:
                tiled[d] = spmm_mod.TiledSpmmPlan(ip, ix, v, n, n, dim=d)
    ip_full_h = ip.cpu().numpy() if rank == 0 else None

    def step(record=None):
        # the products of a step are independent: all their exchanges are started first (on the
        # library's communication stream), and each SpMM waits only for its own operand, slice by slice
        # (four exchange slots: widths are taken four at a time)
        for g0 in range(0, len(dims), 4):
            group = list(enumerate(dims))[g0:g0 + 4]
            if world > 1:
                for di, d in group:
                    shard_of[d].gather_begin(xs[d], slot=di % 4)
            for di, d in group:
                if record is not None:
                    record[di][0].record()
                if d in tiled:
                    tiled[d].run(xs[d], ys[d])
                elif world > 1:
                    shard_of[d].multiply(ys[d], slot=di % 4)
                else:
                    shard.step(xs[d], ys[d])
                if record is not None:
                    record[di][1].record()

    def count_launches():
        total = 0
        for di, d in enumerate(dims):
            if d in tiled:
                tiled[d].run(xs[d], ys[d]); total += tiled[d].info()["launches_last_run"]
            elif world > 1:
                shard_of[d].gather_begin(xs[d], slot=di % 4); shard_of[d].multiply(ys[d], slot=di % 4)
                total += shard_of[d].info()["launches_last_step"]
            else:
                shard.step(xs[d], ys[d]); total += shard.info()["launches_last_step"]
        return total

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    launches_per_step = count_launches()
    barrier()
    # the step's results against the fp64 product, once, before anything is timed
    verified = checksum_check(ip, ix, v, n, xs_full, ys, shard_of, col_of, dims, dev, world)
    del xs_full
    if world > 1:
        del ip, ix, v
    torch.cuda.empty_cache()
    barrier()

    uuid = str(getattr(torch.cuda.get_device_properties(dev), "uuid", ""))
    sampler = ClockSampler(uuid)
    evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in dims]
           for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for k in range(args.steps):
        step(evs[k])
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # keep the same load running (untimed) until the clock sampler has seen about 1.5 s of it; the
    # number of extra steps comes from the reduced time, so every rank runs the same collectives
    for _ in range(int(max(0.0, 1500.0 - float(t.item())) / max(float(t.item()) / args.steps, 1e-3))):
        step()
    torch.cuda.synchronize(dev)
    clocks = sampler.stop()
    per_dim_ms = torch.tensor([np.mean([evs[k][di][0].elapsed_time(evs[k][di][1]) for k in range(args.steps)])
                               for di in range(len(dims))], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(per_dim_ms, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    per_dim_ms = per_dim_ms.tolist()
    flops_step = 2.0 * nnz * sum(dims)
    value = flops_step * args.steps / (total_ms / 1e3) / 1e9

    # where the time goes on several GPUs: the same products with nothing exchanged (the operand of
    # the previous step is still in the slots), and the exchanges alone
    multi = None
    if world > 1:
        def timed_loop(fn, reps=10):
            fn(); barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record(); barrier()
            tt = torch.tensor([a.elapsed_time(b) / reps], dtype=torch.float64, device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return float(tt.item())

        def only_products():
            for di, d in list(enumerate(dims))[-4:]:        # the operands still in the four slots
                shard_of[d].multiply(ys[d], slot=di % 4)

        def only_exchanges():
            for di, d in list(enumerate(dims))[-4:]:
                shard_of[d].gather_begin(xs[d], slot=di % 4)
            for di, d in list(enumerate(dims))[-4:]:
                shard_of[d].wait_gathered(slot=di % 4)

        compute_ms = timed_loop(only_products)
        exchange_ms = timed_loop(only_exchanges)
        nnz_local = torch.tensor([shard.local_nnz], dtype=torch.float64, device=dev)
        nnz_max = nnz_local.clone(); dist.all_reduce(nnz_max, op=dist.ReduceOp.MAX)
        multi = {"step_ms": total_ms / args.steps, "products_without_exchange_ms": compute_ms,
                 "exchanges_without_products_ms": exchange_ms, "exchange": "ncclAllGather inside the library",
                 "step_minus_products_ms": total_ms / args.steps - compute_ms,
                 "exchange_slices": {str(d): shard_of[d].slices for d in dims},
                 "column_ranges": {str(d): ranges_of[d] for d in dims},
                 "feature_groups": {str(d): (fg if d in fg_dims else 1) for d in dims},
                 "rows_per_block": {str(d): shard_of[d].rows_per_block for d in dims},
                 "max_local_nnz_over_mean": float(nnz_max.item()) * world / nnz,
                 "exchanged_bytes_in_per_rank_per_step": sum(4 * (col_of[d][1] - col_of[d][0]) * shard_of[d].rows_per_block
                                                             * (shard_of[d].world - 1) for d in dims),
                 "limiting_phase": "products" if compute_ms > 0.5 * total_ms / args.steps else "exchange"}

    if args.kernel_only:
        # profiling mode: the resident-data loop only (no end-to-end, CPU or reference legs)
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "steps": args.steps,
                              "ms_per_step": total_ms / args.steps, "dims": list(dims), "per_dim_ms": per_dim_ms, "kernel_only": True,
                              "tiled_dims": sorted(tiled), "multi_gpu": multi, "verified": verified}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end through the host-buffer C-ABI calls, pinned host memory --------------------
    # every rank's inputs are its block of A (.block4, renamed column ids, values: rebuilt on the host
    # from the same layout) and the whole X; its outputs are its rows of Y
    host = spmm_mod.HostSpmm()
    n_rows_host, n_cols_host = n, n
    if world == 1:
        from accelgcn import partition
        hb = {"b4": partition.block_level_partition_device(ip).cpu().pin_memory(), "ix": ix.cpu().pin_memory(),
              "v": v.cpu().pin_memory()}
        hx = {d: xs[d].cpu().pin_memory() for d in dims}
    e2e = None
    if world == 1:
        hy = {d: torch.empty((n_rows_host, d), dtype=torch.float32).pin_memory() for d in dims}
        e2e_steps = max(1, min(args.steps, 5))

        def e2e_step(with_graph=True):
            # every input of the step crosses PCIe once: with_graph -> .block4, column ids and values too
            if with_graph:
                host.step_batch(hb["b4"], hb["ix"], hb["v"], [hx[d] for d in dims], n_rows_host, outs=[hy[d] for d in dims])
            else:
                host.run_batch([hx[d] for d in dims], outs=[hy[d] for d in dims])

        step_ms = []

        def timed(fn, reps):
            fn()
            barrier()
            t0 = time.perf_counter()
            for _ in range(reps):
                t1 = time.perf_counter()
                fn()                                  # returns when the step's last Y is in host memory
                step_ms.append((time.perf_counter() - t1) * 1e3)
            barrier()
            return time.perf_counter() - t0

        e2e_s = timed(e2e_step, e2e_steps)
        e2e_timing = host.last_timing()           # where the time of the last streamed call went (ms from its first upload)
        e2e_step_ms = list(step_ms)
        e2e_ok = all(bool(torch.equal(hy[d], ys[d].cpu())) for d in dims if d not in tiled)
        resident_s = timed(lambda: e2e_step(False), e2e_steps)           # graph uploaded once, at set-up
        e2e_ok = e2e_ok and all(bool(torch.equal(hy[d], ys[d].cpu())) for d in dims if d not in tiled)
        pcie = pcie_peaks(dev)
        graph_bytes = 16 * int(hb["b4"].shape[0]) + 8 * nnz
        h2d = graph_bytes + sum(4 * d * n_cols_host for d in dims)
        d2h = sum(4 * d * n_rows_host for d in dims)
        e2e = {"value": flops_step * e2e_steps / e2e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "steps": e2e_steps, "ms_per_step": e2e_s / e2e_steps * 1e3,
               "pcie_gbs_up": h2d / (e2e_s / e2e_steps) / 1e9, "pcie_measured_peaks": pcie,
               "frac_of_h2d_floor": (h2d / (pcie["h2d_gbs"] * 1e9)) / (e2e_s / e2e_steps),
               "call": "agcn_spmm_host_batch: graph and X up, Y down, A multiplied range by range as it arrives",
               "bit_identical_to_resident_run": e2e_ok, "last_call_ms": e2e_timing, "each_step_ms": e2e_step_ms,
               "graph_resident": {"value": flops_step * e2e_steps / resident_s / 1e9, "unit": UNIT,
                                  "ms_per_step": resident_s / e2e_steps * 1e3,
                                  "h2d_bytes_per_step": h2d - graph_bytes, "d2h_bytes_per_step": d2h,
                                  "call": "agcn_host_spmm_batch",
                                  "note": "graph uploaded once at set-up (SPMM_BASE constructor), X and Y cross PCIe every step"}}
    host.close()
    if world > 1:
        e2e = e2e_sharded(args, shard_of, xs, ys, dims, dev, world, barrier, flops_step)
    gcn_rec = None
    if args.workload == "cfg2" and not args.no_gcn:
        gcn_rec = gcn_subrecord(rank, world, dev, barrier)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = hbm_peak()
    props = torch.cuda.get_device_properties(dev)
    sm_mhz = clocks["sm_mhz"] or clocks["sm_max_mhz"] or 1965.0
    fp32_peak = props.multi_processor_count * 128 * 2 * sm_mhz * 1e6
    l2_peaks = gather_peaks(dims) if world == 1 else {}
    per_dim = []
    for d, ms in zip(dims, per_dim_ms):
        b = min_bytes(nnz, n_blocks, n, n, d)
        t_hbm, t_fp32 = b / (peak * 1e9) * 1e3, 2.0 * nnz * d / fp32_peak * 1e3
        gather_gbs = (nnz * (8 + 4 * d) + 4 * d * n + 16 * n_blocks) / ms / 1e6
        row = {"dim": d, "ms": ms, "gflops": 2.0 * nnz * d / ms / 1e6, "hbm_gbs": b / ms / 1e6,
               "hbm_frac": b / ms / 1e6 / peak, "t_bound_ms": max(t_hbm, t_fp32),
               "bound_term": "hbm" if t_hbm >= t_fp32 else "fp32", "frac_of_t_bound": max(t_hbm, t_fp32) / ms,
               "gather_gbs_l2_inclusive": gather_gbs, "kernel": "column-tiled" if d in tiled else "one launch set"}
        if d in l2_peaks:
            row["l2_gather_peak_gbs"] = l2_peaks[d]
            row["gather_frac_of_measured_l2_peak"] = gather_gbs / l2_peaks[d]
        per_dim.append(row)
    top = max(per_dim, key=lambda r: r["ms"])
    variant = "column-tiled" if top["dim"] in tiled else ("two 64-column passes" if top["dim"] > 64 else "one pass")
    if world > 1:
        variant = (f"{fg} feature groups of {world // fg} row blocks" if top["dim"] in fg_dims
                   else "row blocks, column ranges" if ranges_of[top["dim"]] != 1 else "row blocks")
    traffic = NCU_TRAFFIC_BYTES.get((args.workload, top["dim"], variant)) if world == 1 else None
    # `bound`/`achieved`/`frac` follow the contract: compulsory HBM bytes per launch over the CUDA-event
    # time against the measured copy bandwidth.  Which resource really binds is named beside it.
    roofline = {"bound": "hbm", "achieved": top["hbm_gbs"], "peak": peak, "unit": "GB/s",
                "frac": top["hbm_frac"], "traffic": traffic, "kernel": f"spmm_units_kernel dim={top['dim']} ({variant})",
                "peak_source": peak_src,
                "algorithmic_bytes_per_launch": min_bytes(nnz, n_blocks, n, n, top["dim"]),
                "binding_term_of_max_hbm_fp32": top["bound_term"], "frac_of_t_bound": top["frac_of_t_bound"],
                "fp32_frac_at_sampled_clock": 2.0 * nnz * top["dim"] / (top["ms"] / 1e3) / fp32_peak,
                "l2_gather_peak_gbs": top.get("l2_gather_peak_gbs"),
                "gather_frac": top.get("gather_frac_of_measured_l2_peak"),
                "note": "the gather moves nnz*4*dim bytes of X through L2 for 4*dim*N bytes from HBM; "
                        "gather_frac = L2-inclusive bytes per second over the measured L2 gather rate of this GPU"}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_description(args.workload, g.info, n, nnz, n_blocks, dims),
            "roofline": roofline, "per_dim": per_dim, "clocks": clocks, "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps, "verified": verified,
            "plan": shard.info(), "preprocess_ms": g.info.get("preprocess_ms")}
    if multi is not None:
        line["multi_gpu"] = multi
    if gcn_rec is not None:
        line["gcn"] = gcn_rec

    if world == 1:
        ip_h, ix_h, v_h = ip_full_h, ix.cpu().numpy(), v.cpu().numpy()
        xs_h = [xs[d].cpu().numpy() for d in dims]
        if not args.no_ref_gpu:
            from accelgcn import partition
            b4_h = partition.block_level_partition_device(ip).cpu().numpy()
            line["reference_gpu"] = reference_gpu_kernels(b4_h, ip_h, ix_h, v_h, xs_h, dims, nnz)
        from oracle import oracle
        gf, dt, desc, stride = cpu_spmm_rate(ip_h, ix_h, v_h, xs_h, args.cpu_seconds)
        line["cpu_baseline"] = {"value": gf, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
                                "sample": desc, "seconds": dt,
                                "reference_cpu_path": cpu_reference_extras(ip_h, ix_h, v_h, xs_h, stride)}
    else:
        dist.destroy_process_group()
    print(json.dumps(line), flush=True)


def gcn_subrecord(rank, world, dev, barrier, workload="cfg5-5m", steps=5):
    """A short run of the configuration-5 forward (N = 5e6) inside the default line, so that a scaling run of
    the default workload also carries the forward at every GPU count: ms per forward, the per-layer split,
    the sampled fp64 check.  `python bench.py --workload cfg5[-5m]` is the full record of the same path."""
    import torch
    import torch.distributed as dist
    from accelgcn import synth, sharded, gcn

    g, ip, ix, v, _dims = build_workload(workload, dev)
    n, nnz, seed = g.n, int(ix.numel()), g.info["seed"]
    del g
    shard = sharded.ShardedSpmm(ip, ix, v, rank, world)

    def x_rows(rows):
        out = torch.empty((rows.numel(), 128), dtype=torch.float32, device=dev)
        for a in range(0, rows.numel(), 2_000_000):
            r = rows[a:a + 2_000_000]
            base = (r * 128).unsqueeze(1) + torch.arange(128, device=dev, dtype=torch.int64)
            out[a:a + r.numel()] = synth.uniform_f32_at(seed, 7, base.reshape(-1), -1.0, 1.0).reshape(-1, 128)
        return out
    x_block = shard.to_block(x_rows)
    w1, w2 = synth.glorot(128, 128, seed, 8, dev), synth.glorot(128, 128, seed, 9, dev)
    fwd = gcn.GcnForward(shard, [w1, w2])
    out = torch.empty_like(x_block)
    for _ in range(3):
        fwd.forward(x_block, out=out)
    barrier()
    fwd.status()
    sampled = gcn_sampled_check(ip, ix, v, x_rows, w1, w2, out, shard.rows_of(), dev, n_sample=16)
    ok = torch.tensor([1.0 if sampled["ok"] else 0.0], device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps):
        fwd.forward(x_block, out=out)
    e1.record()
    barrier()
    parts = torch.tensor(np.asarray(fwd.status(timings=True)).reshape(-1), dtype=torch.float64, device=dev)
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(parts, op=dist.ReduceOp.MAX)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    p = parts.tolist()
    ms = float(t.item()) / steps
    per_layer = {"gemm": (p[0] + p[3]) / 2, "wait_for_exchange": (p[1] + p[4]) / 2, "spmm_relu": (p[2] + p[5]) / 2}
    rec = {"workload": f"{workload}: two-layer GCN forward, N={n}, nnz={nnz}, 128 features, through agcn_gcn2_forward_*",
           "steps": steps, "warmup": 3, "ms_per_forward": ms,
           "gflops": 2 * (2.0 * nnz * 128 + 2.0 * n * 128 * 128) / ms / 1e6, "per_layer_ms": per_layer,
           "limiting_phase": max(per_layer.items(), key=lambda kv: kv[1])[0],
           "exchanged_bytes_in_per_rank_per_layer": 4 * 128 * shard.rows_per_block * (world - 1),
           "sampled_rows_check_ok_on_every_rank": bool(ok.item() > 0), "sampled_rows_check": sampled,
           "gpu_launches_per_forward": 2 * (1 + shard.info()["launches_last_step"])}
    fwd.close()
    shard.close()
    return rec


def e2e_sharded(args, shard_of, xs, ys, dims, dev, world, barrier, flops_step):
    """End to end on several GPUs: every rank's block rows of X go up from pinned host memory, the
    step (exchange + products) runs, its block rows of Y come down -- all inside the timed region.
    Three streams: each upload is followed, on the upload stream, by the start of its exchange; the
    products run on the current stream, each waiting for its own operand only; every result goes down
    on a third stream while the next product runs."""
    import torch
    import torch.distributed as dist
    hx = {d: xs[d].cpu().pin_memory() for d in dims}
    hy = {d: torch.empty(tuple(ys[d].shape), dtype=torch.float32).pin_memory() for d in dims}
    xd = {d: torch.empty_like(xs[d]) for d in dims}
    cur = torch.cuda.current_stream(dev)
    s_up, s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    done = {d: torch.cuda.Event() for d in dims}

    def step():
        for g0 in range(0, len(dims), 4):
            group = list(enumerate(dims))[g0:g0 + 4]
            s_up.wait_stream(cur)                   # the slots' previous readers are behind this point
            with torch.cuda.stream(s_up):
                for di, d in group:
                    xd[d].copy_(hx[d], non_blocking=True)
                    shard_of[d].gather_begin(xd[d], slot=di % 4, stream=s_up)
            for di, d in group:
                shard_of[d].multiply(ys[d], slot=di % 4, stream=cur)
                done[d].record(cur)
                s_down.wait_event(done[d])
                with torch.cuda.stream(s_down):
                    hy[d].copy_(ys[d], non_blocking=True)
        torch.cuda.synchronize(dev)

    reps = max(1, min(args.steps, 5))
    step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(reps):
        step()
    barrier()
    dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
    dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    same = all(bool(torch.equal(hy[d], ys[d].cpu())) for d in dims)
    return {"value": flops_step * reps / float(dt.item()) / 1e9, "unit": UNIT,
            "h2d_bytes_per_step": sum(4 * xs[d].numel() for d in dims), "d2h_bytes_per_step": sum(4 * ys[d].numel() for d in dims),
            "steps": reps, "ms_per_step": float(dt.item()) / reps * 1e3, "bit_identical_to_resident_run": same,
            "call": "per rank: block rows of X up, agcn_dist_gather_begin + agcn_dist_spmm_gathered, block rows of Y down "
                    "(each rank's block of A is resident); uploads, products and downloads on three streams"}


def ours_gcn(args, rank, world, local_rank):
    """Two-layer GCN forward on the row-sharded operator (configuration 5) through agcn_gcn2_forward_*.
    One step = one forward: per layer a TF32 GEMM on the owned rows, the all-gather of the result, the
    SpMM with fused ReLU."""
    import torch
    import torch.distributed as dist
    from accelgcn import synth, sharded, gcn, _lib

    assert torch.cuda.is_available(), "bench.py needs a CUDA device: the library has no CPU fallback"
    _lib.load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()

    g, ip, ix, v, _dims = build_workload(args.workload, dev)
    n, nnz, seed, info = g.n, int(ix.numel()), g.info["seed"], dict(g.info)
    del g
    shard = sharded.ShardedSpmm(ip, ix, v, rank, world, exchange_slices=args.slices if world > 1 else 1)
    ip_h = ip.cpu().numpy() if rank == 0 and world == 1 else None
    ip_keep, ix_keep, v_keep = ip, ix, v            # the whole matrix, kept until the sampled check below
    del ip, ix, v
    per = shard.rows_per_block
    nb = torch.tensor([int(shard.n_blocks)], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(nb)
    n_blocks = int(nb.item())
    # this rank's block rows of X, generated row by row (the generator addresses elements by index)
    def x_rows(rows):
        out = torch.empty((rows.numel(), 128), dtype=torch.float32, device=dev)
        for a in range(0, rows.numel(), 2_000_000):
            r = rows[a:a + 2_000_000]
            base = (r * 128).unsqueeze(1) + torch.arange(128, device=dev, dtype=torch.int64)
            out[a:a + r.numel()] = synth.uniform_f32_at(seed, 7, base.reshape(-1), -1.0, 1.0).reshape(-1, 128)
        return out
    x_block = shard.to_block(x_rows)
    w1, w2 = synth.glorot(128, 128, seed, 8, dev), synth.glorot(128, 128, seed, 9, dev)
    fwd = gcn.GcnForward(shard, [w1, w2])
    out = torch.empty_like(x_block)

    for _ in range(max(args.warmup, 3)):
        fwd.forward(x_block, out=out)
    barrier()
    fwd.status()
    sampled = gcn_sampled_check(ip_keep, ix_keep, v_keep, x_rows, w1, w2, out, shard.rows_of(), dev)
    if world > 1:
        flag = torch.tensor([1.0 if sampled["ok"] else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        sampled["ok_on_every_rank"] = bool(flag.item() > 0)
        ip_keep = ix_keep = v_keep = None
        torch.cuda.empty_cache()
    barrier()
    uuid = str(getattr(torch.cuda.get_device_properties(dev), "uuid", ""))
    sampler = ClockSampler(uuid)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    parts_sum = np.zeros(6)
    barrier()
    e0.record()
    for _ in range(args.steps):
        fwd.forward(x_block, out=out)
    e1.record()
    barrier()
    parts_sum += np.asarray(fwd.status(timings=True)).reshape(-1)       # the last forward's split
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    for _ in range(int(max(0.0, 1500.0 - float(t.item())) / max(float(t.item()) / args.steps, 1e-3))):
        fwd.forward(x_block, out=out)           # same count on every rank (it comes from the reduced time)
    torch.cuda.synchronize(dev)
    clocks = sampler.stop()
    parts = torch.tensor(parts_sum, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(parts, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    p = parts.tolist()
    gemm_ms, gather_ms, spmm_ms = (p[0] + p[3]) / 2, (p[1] + p[4]) / 2, (p[2] + p[5]) / 2
    flops_step = 2 * (2.0 * nnz * 128 + 2.0 * n * 128 * 128)
    value = flops_step * args.steps / (total_ms / 1e3) / 1e9
    per_layer = {"gemm": gemm_ms, "wait_for_first_exchanged_slice": gather_ms, "spmm_relu_incl_later_slices": spmm_ms,
                 "exchange_slices": shard.slices,
                 "exchanged_bytes_in_per_rank_per_layer": 4 * 128 * per * (world - 1),
                 "limiting_phase": max((("gemm", gemm_ms), ("exchange", gather_ms), ("spmm", spmm_ms)), key=lambda kv: kv[1])[0]}

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "steps": args.steps,
                              "ms_per_step": total_ms / args.steps, "kernel_only": True, "per_layer_ms": per_layer}))
        if world > 1:
            dist.destroy_process_group()
        return

    # end to end: block rows of X up from pinned host memory, forward, block rows of the output down
    # (the device buffers of the resident run are reused: at N = 5e7 a second set would not fit)
    hx = x_block.cpu().pin_memory()
    hy = torch.empty((per, 128), dtype=torch.float32).pin_memory()
    resident_sum = float(out.sum(dtype=torch.float64))

    def e2e_step():
        x_block.copy_(hx, non_blocking=True)
        hy.copy_(fwd.forward(x_block, out=out), non_blocking=True)
        torch.cuda.synchronize(dev)

    e2e_steps = max(1, min(args.steps, 3))
    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_value = flops_step * e2e_steps / float(e2e_s.item()) / 1e9
    # the end-to-end forward recomputed `out` from the re-uploaded X: same bits give the same fp64 sum; and
    # the downloaded copy equals the device result (compared on the first and last million rows)
    k = min(per, 1_000_000)
    same = bool(float(out.sum(dtype=torch.float64)) == resident_sum and torch.equal(hy[:k], out[:k].cpu())
                and torch.equal(hy[-k:], out[-k:].cpu()))
    if rank != 0:
        dist.destroy_process_group()
        return

    peak, peak_src = hbm_peak()
    gemm_bytes = 2 * 4 * 128 * per + 4 * 128 * 128                       # H read + Z written (+ W)
    spmm_bytes = min_bytes(int(shard.local_nnz), int(shard.n_blocks), per, shard.n_gathered, 128)
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 (SpMM), tf32 multiply / f32 accumulate (X*W)",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: two-layer GCN forward relu(A relu(A X W1) W2) on synthetic config 5, "
                                   f"N={n}, nnz={nnz}, max degree {info['max_degree']}, {n_blocks} .block4 tuples, 128 features, "
                                   f"A in row blocks (equal rows and nonzeros) over {world} GPU(s), all-gather of X*W per layer",
                       "n": n, "nnz": nnz, "n_blocks": n_blocks, "l2": "no flush: every operand is larger than L2"},
            "per_layer_ms": per_layer,
            "roofline": {"bound": "hbm", "achieved": spmm_bytes / spmm_ms / 1e6, "peak": peak, "unit": "GB/s",
                         "frac": spmm_bytes / spmm_ms / 1e6 / peak, "traffic": None, "peak_source": peak_src,
                         "kernel": "spmm_units_kernel dim=128 (+ReLU), per rank",
                         "algorithmic_bytes_per_launch": spmm_bytes,
                         "gemm": {"kernel": "gemm_tf32_128_kernel", "achieved": gemm_bytes / gemm_ms / 1e6,
                                  "frac": gemm_bytes / gemm_ms / 1e6 / peak, "algorithmic_bytes_per_launch": gemm_bytes}},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * 128 * per, "d2h_bytes_per_step": 4 * 128 * per,
                    "steps": e2e_steps, "bit_identical_to_resident_run": same},
            "gpu_launches": args.steps * 2 * (1 + shard.info()["launches_last_step"]),
            "plan": shard.info(), "preprocess_ms": info.get("preprocess_ms"), "sampled_rows_check": sampled}
    if world == 1:
        # CPU baseline on a bounded sample: every k-th row of A (SpMM) and of H (X*W, numpy/BLAS)
        from oracle import oracle
        ix_h, v_h = ix_keep.cpu().numpy(), v_keep.cpu().numpy()
        x_h = x_block[:n].cpu().numpy()           # one rank: block rows are the matrix rows
        gf, dt, desc, stride = cpu_spmm_rate(ip_h, ix_h, v_h, [x_h], args.cpu_seconds)
        rows = x_h[::stride]
        t0 = time.perf_counter()
        rows @ w1.cpu().numpy()
        dt_g = time.perf_counter() - t0
        samp_flops = 2.0 * (nnz / stride) * 128 + 2.0 * len(rows) * 128 * 128
        line["cpu_baseline"] = {"value": samp_flops / (dt + dt_g) / 1e9, "unit": UNIT, "cores": oracle.num_threads(),
                                "kind": "port", "sample": "one layer (X*W then A*Z) on " + desc, "seconds": dt + dt_g}
    else:
        dist.destroy_process_group()
    print(json.dumps(line), flush=True)


def gcn_sampled_check(ip, ix, v, x_rows, w1, w2, out_block, block_rows, dev, n_sample=48):
    """Parity at sizes no CPU forward can check: for a sample of this rank's output rows the whole
    two-hop computation is redone in fp64 on the device from the CSR arrays of the whole matrix
    (block_rows maps local rows to matrix rows).  Rows of more than 2000 nonzeros are left out of the
    sample to keep its two-hop fan-out bounded."""
    import torch
    valid = torch.nonzero(block_rows >= 0).reshape(-1)
    cand = torch.unique(torch.cat([valid[torch.randint(0, valid.numel(), (n_sample,), device=dev)], valid[:1], valid[-1:]]))
    w1d, w2d = w1.double(), w2.double()

    def neighbours(r):
        a, b = int(ip[r]), int(ip[r + 1])
        return ix[a:b].long(), v[a:b].double()

    worst, used = 0.0, 0
    scale = float(out_block.abs().max())
    for j in cand.tolist():
        r = int(block_rows[j])
        c1, a1 = neighbours(r)
        if c1.numel() > 2000:
            continue
        h1 = torch.zeros((c1.numel(), 128), dtype=torch.float64, device=dev)
        for k, col in enumerate(c1.tolist()):
            c2, a2 = neighbours(col)
            if c2.numel() > 200_000:
                break
            h1[k] = torch.clamp((a2[:, None] * (x_rows(c2).double() @ w1d)).sum(0), min=0)
        else:
            ref = torch.clamp((a1[:, None] * (h1 @ w2d)).sum(0), min=0)
            worst = max(worst, float((out_block[j].double() - ref).abs().max()))
            used += 1
    return {"rows_checked": used, "max_abs_err": worst, "output_scale": scale, "tolerance": 4e-3 * scale,
            "ok": bool(used > 0 and worst <= 4e-3 * scale),
            "what": "two-hop fp64 recomputation of sampled output rows on the device; tolerance 4e-3 of the output scale (TF32 dense transform)"}


def ours_replicas(args):
    """SpMM on degree-sequence replicas of the reference's own benchmark graphs, one width, beside the
    reference's kernel and its cuSPARSE call on the same arrays.  Also re-checks that the GPU
    partitioner reproduces every golden .block4 file (SHA-256) on the way."""
    import hashlib
    import torch
    from accelgcn import synth, partition, spmm as spmm_mod, _lib
    from oracle import oracle
    assert torch.cuda.is_available(), "bench.py needs a CUDA device: the library has no CPU fallback"
    _lib.load()
    dev = torch.device("cuda", 0)
    dim = args.dim
    with open(os.path.join(ROOT, "tests", "golden", "block4_kat.json")) as fh:
        kat = json.load(fh)
    rows, tot_flops, tot_ms, launches = [], 0.0, 0.0, 0
    for gi, (name, e) in enumerate(sorted(kat.items())):
        deg = np.concatenate([np.zeros(e["leading_zero_rows"], dtype=np.int64),
                              np.repeat(np.asarray(e["degrees"], dtype=np.int64), np.asarray(e["counts"], dtype=np.int64))])
        n, nnz = len(deg), int(deg.sum())
        ip_h = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
        ip = torch.from_numpy(ip_h).to(dev)
        ix = synth.uniform_int(2000 + gi, 1, 0, nnz, n, dev).to(torch.int32)
        v = 1.0 - synth.uniform_f32(2000 + gi, 2, 0, nnz, 0.0, 1.0, dev)
        x = synth.features(n, dim, 2000 + gi, dev)
        b4 = partition.block_level_partition_device(ip)
        golden = hashlib.sha256(b4.cpu().numpy().tobytes()).hexdigest() == e["sha256"]
        plan = spmm_mod.SpmmPlan(b4, ix, n, n)
        y = torch.empty((n, dim), dtype=torch.float32, device=dev)
        for _ in range(max(args.warmup, 3)):
            plan.run(ix, v, x, y)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            plan.run(ix, v, x, y)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        launches += args.steps * plan.info()["launches_last_run"]
        plan.close()
        row = {"graph": name, "n": n, "nnz": nnz, "n_blocks": int(b4.shape[0]), "block4_matches_golden": golden,
               "ms": ms, "gflops": 2.0 * nnz * dim / ms / 1e6,
               "hbm_frac": min_bytes(nnz, int(b4.shape[0]), n, n, dim) / ms / 1e6 / hbm_peak()[0]}
        if oracle.ref_available() and not args.no_ref_gpu and n * dim < 2**31:
            ix_h, v_h, x_h, b4_h = ix.cpu().numpy(), v.cpu().numpy(), x.cpu().numpy(), b4.cpu().numpy()
            ref = oracle.ref_accel_spmm(b4_h, ip_h, ix_h, v_h, x_h)
            err = np.abs(y.cpu().numpy() - ref)
            row["max_abs_diff_vs_reference_kernel"] = float(err.max())
            row["accel_ms"] = oracle.ref_accel_spmm(b4_h, ip_h, ix_h, v_h, x_h, timing=True) * 1e3
            row["cusparse_ms"] = oracle.ref_cusparse_spmm(ip_h, ix_h, v_h, x_h, timing=True) * 1e3
            if args.gnna and nnz <= 3_000_000:
                # the reference's third kernel (spmm_gnna.cu, timed at main.cu:164-165); it ignores the values of A
                row["gnna_ms"] = oracle.ref_gnna_time(ip_h, ix_h, v_h, x_h) * 1e3
        rows.append(row)
        tot_flops += 2.0 * nnz * dim
        tot_ms += ms
        del ip, ix, v, x, y, b4
        torch.cuda.empty_cache()
    line = {"metric": METRIC, "value": tot_flops / tot_ms / 1e6, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": tot_ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"replicas: degree-sequence replicas of the 16 reference graphs with shipped .block4 files, "
                                   f"uniform random columns, SpMM at dim {dim}; one step = all 16 graphs",
                       "dim": dim, "l2": "small graphs fit L2; no flush (the reference's protocol does not flush either)"},
            "graphs": rows, "gpu_launches": launches}
    have = [r for r in rows if "accel_ms" in r]
    if have:
        line["geomean_speedup_vs_reference_kernel"] = float(np.exp(np.mean([np.log(r["accel_ms"] / r["ms"]) for r in have])))
        line["geomean_speedup_vs_cusparse"] = float(np.exp(np.mean([np.log(r["cusparse_ms"] / r["ms"]) for r in have])))
    print(json.dumps(line), flush=True)


def reference_gpu_kernels(block4, ip_h, ix_h, v_h, xs_h, dims, nnz):
    """The reference's own spmm_accel kernel and its cuSPARSE call, compiled from the reference
    sources (oracle/_ref), timed on this GPU with the reference's own protocol (mean wall-clock
    seconds of 4 resp. 10 launches after as many warm-ups)."""
    from oracle import oracle
    if not oracle.ref_available():
        return {"unavailable": "oracle/_ref/libref_accel.so not built (needs the reference tree at build time)"}
    out = {}
    for x, d in zip(xs_h, dims):
        if (len(ip_h) - 1) * d >= 2**31 or d > 128:
            out[str(d)] = {"unavailable": "outside the reference kernel's int32 / dim <= 128 limits"}
            continue
        ta = oracle.ref_accel_spmm(block4, ip_h, ix_h, v_h, x, timing=True)
        tc = oracle.ref_cusparse_spmm(ip_h, ix_h, v_h, x, timing=True)
        out[str(d)] = {"accel_ms": ta * 1e3, "accel_gflops": 2.0 * nnz * d / ta / 1e9,
                       "cusparse_ms": tc * 1e3, "cusparse_gflops": 2.0 * nnz * d / tc / 1e9}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="cfg2")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="CPU time spent on the cpu_baseline sample")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's GPU kernels")
    ap.add_argument("--feature-groups", type=int, default=0,
                    help="several GPUs: multiply wide operands as this many independent products of dim / F columns, each "
                         "row-sharded over world / F ranks (0 = 4 on eight GPUs, 2 on two or four, else 1)")
    ap.add_argument("--feature-groups-min-dim", type=int, default=128, help="narrowest product that --feature-groups applies to")
    ap.add_argument("--feature-groups-min-width", type=int, default=32, help="narrowest dim / F that --feature-groups applies to")
    ap.add_argument("--no-gcn", action="store_true", help="default workload: leave out the short configuration-5 forward (`gcn` record)")
    ap.add_argument("--dim", type=int, default=64, help="dense width of the replicas workload")
    ap.add_argument("--kernel-only", action="store_true", help="resident-data loop only (for profiling under ncu)")
    ap.add_argument("--slices", type=int, default=1,
                    help="N > 1: exchange the dense operand in this many row slices and multiply slice by slice")
    ap.add_argument("--slices-min-dim", type=int, default=128, help="narrowest width that --slices applies to (SpMM workloads)")
    ap.add_argument("--tiled", choices=("auto", "off"), default="auto",
                    help="one GPU: run products whose X exceeds L2 column-tiled (auto) or never (off)")
    ap.add_argument("--gnna", action="store_true", help="replicas workload: also time the reference's GNNAdvisor kernel")
    ap.add_argument("--dims", type=str, default="", help="comma-separated dense widths instead of the workload's own")
    args = ap.parse_args()
    if args.dims:
        cfg_id, scale, _ = WORKLOADS[args.workload]
        WORKLOADS[args.workload] = (cfg_id, scale, tuple(int(t) for t in args.dims.split(",")))
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and args.workload == "replicas":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the replicas workload has no CPU arm; use a cfg workload"}))
    elif args.impl == "reference":
        reference_arm(args, rank, world)
    elif args.workload == "replicas":
        if rank == 0:
            ours_replicas(args)
    elif args.workload in GCN_WORKLOADS:
        ours_gcn(args, rank, world, local_rank)
    else:
        ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
