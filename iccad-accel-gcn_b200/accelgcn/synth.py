"""Seeded synthetic graphs standing in for the reference's 18-graph benchmark
set (README.md:41-53 -- a download that is not available offline) and for the
five workload configurations this project is measured on.

Everything random comes from a counter-based generator (splitmix64 of
seed/stream/index) and every sampling step is integer arithmetic, so the same
(seed, config) gives bit-identical graphs on the CPU and on a GPU; torch is
used only as the array library that runs on either.  Only the node weights
are floating point, and they are always computed on the host in float64.

A graph is returned in CSR with sorted, duplicate-free columns in its ORIGINAL
node numbering (not degree-ordered): ordering by degree is the job of the
library's degree sort.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np
import torch

_MASK64 = (1 << 64) - 1


def _s64(v: int) -> int:
    """Python int -> the int64 with the same 64-bit pattern."""
    v &= _MASK64
    return v - (1 << 64) if v >= (1 << 63) else v


_GOLDEN = _s64(0x9E3779B97F4A7C15)
_M1 = _s64(0xBF58476D1CE4E5B9)
_M2 = _s64(0x94D049BB133111EB)


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    """Logical right shift of int64 bit patterns."""
    return (x >> s) & ((1 << (64 - s)) - 1)


def splitmix64(seed: int, stream: int, start: int, count: int, device) -> torch.Tensor:
    """count 64-bit outputs (as int64 bit patterns): element k is the splitmix64
    finaliser of  seed + stream * 2^32 * golden + (start + k + 1) * golden."""
    base = _s64(seed + ((stream * 0x100000001B3) & _MASK64))
    idx = torch.arange(start + 1, start + 1 + count, dtype=torch.int64, device=device)
    z = idx * _GOLDEN + base
    z = (z ^ _lsr(z, 30)) * _M1
    z = (z ^ _lsr(z, 27)) * _M2
    return z ^ _lsr(z, 31)


def uniform_f32_at(seed, stream, index: torch.Tensor, lo: float, hi: float) -> torch.Tensor:
    """Elements `index` (int64 tensor, any shape) of the stream uniform_f32(seed, stream, 0, ...) draws from:
    the generator is counter-based, so any subset can be produced without the rest."""
    base = _s64(seed + ((stream * 0x100000001B3) & _MASK64))
    z = (index + 1) * _GOLDEN + base
    z = (z ^ _lsr(z, 30)) * _M1
    z = (z ^ _lsr(z, 27)) * _M2
    r = _lsr(z ^ _lsr(z, 31), 40).to(torch.float32)
    return r * ((hi - lo) / float(1 << 24)) + lo


def uniform_int(seed, stream, start, count, bound: int, device) -> torch.Tensor:
    """Integers in [0, bound) (bound < 2^62); the modulo bias is below 2^-1."""
    r = _lsr(splitmix64(seed, stream, start, count, device), 1)    # 63 random bits, non-negative
    return r % bound


def uniform_f32(seed, stream, start, count, lo: float, hi: float, device) -> torch.Tensor:
    """float32 in [lo, hi): 24 random bits scaled -- exact in fp32 on any device."""
    r = _lsr(splitmix64(seed, stream, start, count, device), 40).to(torch.float32)   # [0, 2^24)
    return r * ((hi - lo) / float(1 << 24)) + lo


@dataclasses.dataclass
class Graph:
    name: str
    n: int
    indptr: torch.Tensor     # int32 [n+1]
    indices: torch.Tensor    # int32 [nnz], sorted within each row
    vals: torch.Tensor       # float32 [nnz]
    info: dict

    @property
    def nnz(self) -> int:
        return int(self.indices.numel())


# --------------------------------------------------------------------------
# node weights (host, float64)
# --------------------------------------------------------------------------
def power_law_weights(n: int, gamma: float, mean: float, max_w: float | None) -> np.ndarray:
    """w_i proportional to (i + i0)^(-1/(gamma-1)), rescaled to the requested mean, capped."""
    alpha = 1.0 / (gamma - 1.0)
    i0 = 1.0
    ranks = np.arange(n, dtype=np.float64) + i0
    w = ranks ** (-alpha)
    for _ in range(60):                      # capping lowers the mean; rescale until it fits
        w *= mean / w.mean()
        if max_w is None or w.max() <= max_w * (1 + 1e-12):
            break
        w = np.minimum(w, max_w)
    return w


def log_normal_weights(n: int, sigma: float, mean: float, seed: int) -> np.ndarray:
    """w_i = exp(mu + sigma z_i), z_i standard normal via the inverse CDF of splitmix64 uniforms."""
    from scipy.special import ndtri
    bits = _lsr(splitmix64(seed, 3, 0, n, "cpu"), 11).numpy().astype(np.float64)   # 53 bits
    u = (bits + 0.5) / float(1 << 53)
    mu = math.log(mean) - 0.5 * sigma * sigma
    return np.exp(mu + sigma * ndtri(u))


def _csr_from_keys(keys: torch.Tensor, n: int):
    """sorted unique (row * n + col) keys -> (indptr int32, indices int32, degrees int64)"""
    rows = torch.div(keys, n, rounding_mode="floor")
    cols = keys - rows * n
    deg = torch.bincount(rows, minlength=n)
    indptr = torch.zeros(n + 1, dtype=torch.int64, device=keys.device)
    torch.cumsum(deg, 0, out=indptr[1:])
    return indptr.to(torch.int32), cols.to(torch.int32), deg


def chung_lu(name: str, n: int, weights: np.ndarray, target_nnz: int, seed: int, device,
             self_loops: bool = True, gcn_values: bool = True) -> Graph:
    """Symmetric Chung-Lu graph by edge sampling: both endpoints of every edge
    are drawn from the weight distribution by inverse CDF on integer-quantised
    cumulative weights, node ids are shuffled by a seeded permutation, the
    edge list is symmetrised, de-duplicated and (optionally) given self loops.
    Edges are over-sampled until the realised nnz is within 5 % of the target."""
    dev = torch.device(device)
    wq = np.maximum(np.rint(weights * (1 << 20) / weights.mean()), 1.0).astype(np.int64)
    cum = torch.cumsum(torch.from_numpy(wq).to(dev), 0)
    total = int(cum[-1].item())
    shuffle = torch.sort(splitmix64(seed, 1, 0, n, dev), stable=True).indices    # position -> node id
    m = max(1, (target_nnz - (n if self_loops else 0)) // 2)
    keys = None
    for attempt in range(6):
        u = shuffle[torch.searchsorted(cum, uniform_int(seed, 10 + 2 * attempt, 0, m, total, dev), right=True)]
        v = shuffle[torch.searchsorted(cum, uniform_int(seed, 11 + 2 * attempt, 0, m, total, dev), right=True)]
        parts = [u * n + v, v * n + u]
        if self_loops:
            ar = torch.arange(n, dtype=torch.int64, device=dev)
            parts.append(ar * n + ar)
        keys = torch.unique(torch.cat(parts))          # sorted
        del u, v, parts
        got = int(keys.numel())
        if got >= 0.95 * target_nnz or attempt == 5:
            break
        m = int(m * min(4.0, 1.08 * target_nnz / max(got, 1))) + 1
    indptr, indices, deg = _csr_from_keys(keys, n)
    if gcn_values:
        # D^-1/2 (A + I) D^-1/2 with D the row degree (self loop included); float64 then rounded once
        d = deg.to(torch.float64).clamp_(min=1.0)
        rows = torch.div(keys, n, rounding_mode="floor")
        vals = (1.0 / torch.sqrt(d[rows] * d[indices.to(torch.int64)])).to(torch.float32)
    else:
        vals = uniform_f32(seed, 5, 0, int(keys.numel()), 0.0, 1.0, dev)
    info = {"target_nnz": int(target_nnz), "sampled_edges": int(m), "max_degree": int(deg.max().item()),
            "zero_degree_rows": int((deg == 0).sum().item())}
    return Graph(name, n, indptr, indices, vals, info)


def skewed_rows(name: str, n: int, gamma: float, max_degree: int, target_nnz: int, seed: int, device) -> Graph:
    """Row-degree-first generator (not symmetrised): row i of a shuffled
    power-law degree sequence draws its columns uniformly, duplicates are
    dropped, values are uniform in (0, 1]."""
    dev = torch.device(device)
    w = power_law_weights(n, gamma, target_nnz / n, float(max_degree))
    deg = np.minimum(np.floor(w + 0.5), max_degree).astype(np.int64)
    deg[0] = max_degree                                   # the configuration fixes the maximum degree
    shuffle = torch.sort(splitmix64(seed, 1, 0, n, dev), stable=True).indices
    deg_t = torch.zeros(n, dtype=torch.int64, device=dev)
    deg_t[shuffle] = torch.from_numpy(deg).to(dev)
    rows = torch.repeat_interleave(torch.arange(n, dtype=torch.int64, device=dev), deg_t)
    cols = uniform_int(seed, 10, 0, int(rows.numel()), n, dev)
    keys = torch.unique(rows * n + cols)
    indptr, indices, d = _csr_from_keys(keys, n)
    vals = 1.0 - uniform_f32(seed, 5, 0, int(keys.numel()), 0.0, 1.0, dev)    # (0, 1]
    info = {"target_nnz": int(target_nnz), "max_degree": int(d.max().item()),
            "zero_degree_rows": int((d == 0).sum().item())}
    return Graph(name, n, indptr, indices, vals, info)


def features(n: int, dim: int, seed: int, device) -> torch.Tensor:
    """Dense X [n x dim] fp32 uniform in [-1, 1) (stream 7 of the seed)."""
    return uniform_f32(seed, 7, 0, n * dim, -1.0, 1.0, torch.device(device)).reshape(n, dim)


def glorot(fan_in: int, fan_out: int, seed: int, stream: int, device) -> torch.Tensor:
    lim = math.sqrt(6.0 / (fan_in + fan_out))
    return uniform_f32(seed, stream, 0, fan_in * fan_out, -lim, lim, torch.device(device)).reshape(fan_in, fan_out)


# --------------------------------------------------------------------------
# the five workload configurations; `scale` shrinks N (and nnz with it) for
# tests that must run in seconds
# --------------------------------------------------------------------------
CONFIGS = {
    1: dict(name="cfg1_powerlaw_16k", seed=1001, n=16_384, mean=8.0, dims=(60,)),
    2: dict(name="cfg2_heavy_250k", seed=1002, n=250_000, mean=490.0, dims=(32, 64, 128)),
    3: dict(name="cfg3_sparse_2m4", seed=1003, n=2_400_000, mean=25.0, dims=(64,)),
    4: dict(name="cfg4_skewed_500k", seed=1004, n=500_000, mean=30.0, dims=tuple(range(16, 129, 4))),
    5: dict(name="cfg5_gcn_50m", seed=1005, n=50_000_000, mean=20.0, dims=(128,)),
}


def make_config(cfg: int, device="cpu", scale: float = 1.0) -> Graph:
    c = CONFIGS[cfg]
    n = max(64, int(round(c["n"] * scale)))
    seed = c["seed"]
    if cfg == 1:
        w = power_law_weights(n, 2.1, c["mean"], None)
        g = chung_lu(c["name"], n, w, int(n * c["mean"]), seed, device)
    elif cfg == 2:
        mean = min(c["mean"], n / 8)
        w = log_normal_weights(n, 1.0, mean, seed)
        g = chung_lu(c["name"], n, w, int(n * mean), seed, device, self_loops=False)
    elif cfg == 3:
        w = power_law_weights(n, 2.3, c["mean"], 20_000.0 * min(1.0, scale * 8))
        g = chung_lu(c["name"], n, w, int(n * c["mean"]), seed, device, self_loops=False)
    elif cfg == 4:
        g = skewed_rows(c["name"], n, 1.8, max(400, int(100_000 * min(1.0, scale * 2))), int(n * c["mean"]), seed, device)
    elif cfg == 5:
        w = power_law_weights(n, 2.2, c["mean"], None)
        g = chung_lu(c["name"], n, w, int(n * c["mean"]), seed, device)
    else:
        raise KeyError(cfg)
    g.info.update(config=cfg, scale=scale, seed=seed)
    if scale != 1.0:
        g.name = f"{g.name}_x{scale:g}"
    return g
