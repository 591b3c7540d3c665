"""Seeded synthetic models and batches with the shapes of the five benchmark configurations.

They stand in for the reference's generated datasets
(data_synthesis/data_generate.py): same kinds of distributions (one-hot,
Poisson and heavy-tailed bag lengths, empty bags, Zipf-like row popularity),
sizes taken from the benchmark definitions.  Everything derives from
`numpy.random.Generator(PCG64(seed))` streams, and table weights come from a
counter-based hash (`synth_rows`) that the CUDA library reproduces bit for bit
(`eb_fill_table`), so any row of any table can be regenerated anywhere without
storing the table.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

WEIGHT_STD = 0.01
_SCALE_DIV = np.float32(37837.227)  # 65536 * sqrt(4 / 12)
_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


# ---------------------------------------------------------------------------
# counter-based weights (bit-identical to eb_fill_kernel)
# ---------------------------------------------------------------------------
def _mix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = x + np.uint64(0x9E3779B97F4A7C15)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))


def synth_rows(seed: int, row_ids: np.ndarray, dim: int, dtype: str = "f32", std: float = WEIGHT_STD) -> np.ndarray:
    """Rows `row_ids` of the synthetic table `seed`: array [len(row_ids), dim] of float32 or float16."""
    row_ids = np.asarray(row_ids, dtype=np.uint64)
    elem = row_ids[:, None] * np.uint64(dim) + np.arange(dim, dtype=np.uint64)[None, :]
    with np.errstate(over="ignore"):
        h = _mix64(np.uint64(seed) * np.uint64(0xD1342543DE82EF95) + elem)
    m = np.uint64(0xFFFF)
    s = ((h & m).astype(np.int64) + ((h >> np.uint64(16)) & m).astype(np.int64)
         + ((h >> np.uint64(32)) & m).astype(np.int64) + ((h >> np.uint64(48)) & m).astype(np.int64) - 131070)
    scale = np.float32(std) / _SCALE_DIV
    w = s.astype(np.float32) * scale
    return w.astype(np.float16) if dtype == "f16" else w


def synth_table(seed: int, rows: int, dim: int, dtype: str = "f32", std: float = WEIGHT_STD) -> np.ndarray:
    """The whole synthetic table (small tables only)."""
    return synth_rows(seed, np.arange(rows, dtype=np.uint64), dim, dtype, std)


# ---------------------------------------------------------------------------
# model description
# ---------------------------------------------------------------------------
@dataclass
class FeatureSpec:
    rows: int
    dim: int
    dtype: str = "f32"                # "f32" | "f16"
    seed: int = 0                     # table seed
    length: str = "onehot"            # onehot | uniform | poisson | powerlaw | empty
    length_args: Tuple = ()           # uniform: (lo, hi); poisson: (mean,); powerlaw: (exponent, max_len, empty_frac)
    index: str = "uniform"            # uniform | zipf
    alpha: float = 1.0                # zipf exponent
    permute: bool = True              # scatter popular rows over the table

    @property
    def row_bytes(self) -> int:
        return self.dim * (2 if self.dtype == "f16" else 4)

    @property
    def table_bytes(self) -> int:
        return self.rows * self.row_bytes


@dataclass
class ModelConfig:
    name: str
    batch: int
    features: List[FeatureSpec] = field(default_factory=list)
    seed: int = 0

    @property
    def output_units(self) -> int:
        return sum(f.dim for f in self.features)

    @property
    def table_bytes(self) -> int:
        return sum(f.table_bytes for f in self.features)


def _log_uniform(rng: np.random.Generator, lo: float, hi: float, n: int) -> np.ndarray:
    return np.exp(rng.uniform(math.log(lo), math.log(hi), n))


def make_config(cfg: int, row_scale: float = 1.0, batch: Optional[int] = None) -> ModelConfig:
    """Benchmark configuration `cfg` (1..5).  `row_scale` < 1 shrinks every table (for CPU-sized tests);
    `batch` overrides the batch size."""
    seed = 1000 + cfg
    rng = np.random.default_rng(seed * 7919)
    feats: List[FeatureSpec] = []

    def rows_scaled(r: float) -> int:
        return max(16, int(r * row_scale))

    if cfg == 1:
        dims = [16, 16, 32, 32, 64, 64, 128, 128]
        for f, d in enumerate(dims):
            feats.append(FeatureSpec(rows=rows_scaled(100_000), dim=d, dtype="f32", seed=seed * 1000 + f,
                                     length="onehot" if f < 2 else "uniform", length_args=() if f < 2 else (1, 20),
                                     index="uniform"))
        return ModelConfig("cfg1-plumbing-8", batch or 256, feats, seed)

    if cfg in (2, 5):
        base_seed = 1002  # cfg5 reuses cfg2's tables
        rng = np.random.default_rng(base_seed * 7919)
        F = 50
        rows = _log_uniform(rng, 1e3, 1e7, F)
        dims = rng.choice([4, 8, 16, 32, 64, 128], F)
        kinds = np.array(["onehot"] * 20 + ["poisson"] * 30)
        rng.shuffle(kinds)
        means = _log_uniform(rng, 2, 100, F)
        for f in range(F):
            feats.append(FeatureSpec(rows=rows_scaled(rows[f]), dim=int(dims[f]), dtype="f32",
                                     seed=base_seed * 1000 + f, length=str(kinds[f]),
                                     length_args=(float(means[f]),) if kinds[f] == "poisson" else (),
                                     index="zipf", alpha=1.05))
        if cfg == 2:
            return ModelConfig("cfg2-hetero-50", batch or 4096, feats, seed)
        # cfg5: shifted inputs on the same tables
        rng5 = np.random.default_rng(seed * 7919)
        group = rng5.permutation(F)
        n10, n01, nempty = int(0.3 * F), int(0.2 * F), int(0.1 * F)
        for k, f in enumerate(group):
            fs = feats[f]
            mean = fs.length_args[0] if fs.length == "poisson" else 1.0
            if k < n10:
                fs.length, fs.length_args = "poisson", (mean * 10.0,)
            elif k < n10 + n01:
                fs.length, fs.length_args = "poisson", (mean * 0.1,)
            elif k < n10 + n01 + nempty:
                fs.length, fs.length_args = "empty", ()
            else:
                fs.index = "uniform"
        return ModelConfig("cfg5-shift-50", batch or 16384, feats, seed)

    if cfg == 3:
        F = 200
        rows = _log_uniform(rng, 1e3, 5e7, F)
        dims = rng.choice([8, 16, 32, 64, 128, 256], F)
        alphas = rng.uniform(0.8, 1.3, F)
        total = float(np.sum(rows * dims * 2))
        rows = rows * (120e9 / total)  # about 120 GB of fp16 tables
        for f in range(F):
            feats.append(FeatureSpec(rows=rows_scaled(max(rows[f], 1e3)), dim=int(dims[f]), dtype="f16",
                                     seed=seed * 1000 + f, length="powerlaw", length_args=(1.5, 500, 0.05),
                                     index="zipf", alpha=float(alphas[f])))
        return ModelConfig("cfg3-heavy-tail-200", batch or 16384, feats, seed)

    if cfg == 4:
        F = 400
        big = 40
        rows = np.concatenate([np.full(big, 1e8), _log_uniform(rng, 1e4, 1e7, F - big)])
        dims = np.concatenate([np.full(big, 64), rng.choice([16, 32, 64, 128], F - big)]).astype(int)
        onehot = rng.random(F) < 0.5
        perm = rng.permutation(F)
        for f in perm:
            feats.append(FeatureSpec(rows=rows_scaled(rows[f]), dim=int(dims[f]), dtype="f16",
                                     seed=seed * 1000 + int(f), length="onehot" if onehot[f] else "poisson",
                                     length_args=() if onehot[f] else (30.0,), index="zipf", alpha=1.1))
        return ModelConfig("cfg4-sharded-400", batch or 65536, feats, seed)

    raise ValueError(f"unknown configuration {cfg}")


# ---------------------------------------------------------------------------
# batches
# ---------------------------------------------------------------------------
def _lengths(fs: FeatureSpec, batch: int, rng: np.random.Generator) -> np.ndarray:
    if fs.length == "onehot":
        return np.ones(batch, dtype=np.int64)
    if fs.length == "empty":
        return np.zeros(batch, dtype=np.int64)
    if fs.length == "uniform":
        lo, hi = fs.length_args
        return rng.integers(lo, hi + 1, batch)
    if fs.length == "poisson":
        return rng.poisson(fs.length_args[0], batch).astype(np.int64)
    if fs.length == "powerlaw":
        expo, max_len, empty_frac = fs.length_args
        pmf = np.arange(1, max_len + 1, dtype=np.float64) ** (-expo)
        cdf = np.cumsum(pmf / pmf.sum())
        lens = np.searchsorted(cdf, rng.random(batch), side="left").astype(np.int64) + 1
        lens = np.minimum(lens, max_len)
        lens[rng.random(batch) < empty_frac] = 0
        return lens
    raise ValueError(fs.length)


def _affine_perm(rows: int, rng: np.random.Generator) -> Tuple[int, int]:
    a = int(rng.integers(1, max(2, rows))) | 1
    while math.gcd(a, rows) != 1:
        a += 2
    return a % rows if rows > 1 else 0, int(rng.integers(0, rows))


def _indices(fs: FeatureSpec, n: int, rng: np.random.Generator) -> np.ndarray:
    if n == 0:
        return np.zeros(0, dtype=np.int64)
    if fs.index == "uniform":
        return rng.integers(0, fs.rows, n)
    # bounded Zipf-like ranks by inverting the continuous power-law CDF on [1, rows + 1)
    u = rng.random(n)
    N = float(fs.rows) + 1.0
    if abs(fs.alpha - 1.0) < 1e-9:
        x = np.exp(u * math.log(N))
    else:
        e = 1.0 - fs.alpha
        x = (u * (N ** e - 1.0) + 1.0) ** (1.0 / e)
    rank = np.clip(x.astype(np.int64) - 1, 0, fs.rows - 1)
    if fs.permute and fs.rows > 1:
        a, b = _affine_perm(fs.rows, np.random.default_rng(fs.seed))
        rank = (rank * a + b) % fs.rows
    return rank


def gen_feature_batch(fs: FeatureSpec, batch: int, seed: int) -> Tuple[np.ndarray, np.ndarray]:
    """(values int64 [nnz], offsets int64 [batch + 1]) of one feature."""
    rng = np.random.default_rng([seed, fs.seed])
    lens = _lengths(fs, batch, rng)
    offsets = np.zeros(batch + 1, dtype=np.int64)
    np.cumsum(lens, out=offsets[1:])
    return _indices(fs, int(offsets[-1]), rng), offsets


def gen_batch(cfg: ModelConfig, seed: int = 0, batch: Optional[int] = None, index_dtype=np.int32):
    """Per-feature lists (values, offsets) of one batch, in `index_dtype`."""
    B = batch or cfg.batch
    vals, offs = [], []
    for fs in cfg.features:
        v, o = gen_feature_batch(fs, B, seed)
        vals.append(v.astype(index_dtype))
        offs.append(o.astype(index_dtype))
    return vals, offs


def pack_batch(values: Sequence[np.ndarray], offsets: Sequence[np.ndarray]) -> Tuple[np.ndarray, np.ndarray]:
    """Per-feature lists -> (values concatenated in feature order, offsets [F, batch + 1])."""
    return np.concatenate(values), np.stack(offsets)


def expected_traffic(cfg: ModelConfig, batch: Optional[int] = None) -> List[float]:
    """Expected gathered bytes per batch of every feature (mean bag length x batch x row bytes): the
    planner's traffic estimate."""
    B = batch or cfg.batch
    out = []
    for fs in cfg.features:
        if fs.length == "onehot":
            mean = 1.0
        elif fs.length == "empty":
            mean = 0.0
        elif fs.length == "uniform":
            mean = (fs.length_args[0] + fs.length_args[1]) / 2.0
        elif fs.length == "poisson":
            mean = fs.length_args[0]
        else:
            expo, max_len, empty_frac = fs.length_args
            l = np.arange(1, max_len + 1, dtype=np.float64)
            pmf = l ** (-expo)
            mean = float((l * pmf).sum() / pmf.sum()) * (1.0 - empty_frac)
        out.append(mean * B * fs.row_bytes)
    return out


def algorithmic_bytes(cfg: ModelConfig, offsets: Sequence[np.ndarray], index_bytes: int = 4) -> int:
    """Roofline numerator of one batch: gathered row bytes + index bytes + offset bytes."""
    total = 0
    for fs, o in zip(cfg.features, offsets):
        nnz = int(o[-1])
        total += nnz * fs.row_bytes + nnz * index_bytes + len(o) * index_bytes
    return total


def sampled_cells(cfg: ModelConfig, values: Sequence[np.ndarray], offsets: Sequence[np.ndarray], n: int,
                  seed: int = 0, features: Optional[Sequence[int]] = None):
    """`n` random (sample, feature) cells of one batch with what they must pool to: yields
    (sample, position of the feature in `features`, expected fp32 vector, sum of magnitudes).  The expected vector is
    the float64 sum of the bag's rows regenerated from the counter-based weights (no table is stored), rounded to
    fp32; an empty bag gives zeros.  `values` / `offsets` are per-feature lists aligned with `features` (default:
    all)."""
    feats = list(range(len(cfg.features))) if features is None else list(features)
    rng = np.random.default_rng(seed)
    batch = len(offsets[0]) - 1
    for _ in range(n):
        k = int(rng.integers(0, len(feats)))
        b = int(rng.integers(0, batch))
        fs = cfg.features[feats[k]]
        idx = np.asarray(values[k][int(offsets[k][b]):int(offsets[k][b + 1])], dtype=np.int64)
        if len(idx) == 0:
            yield b, k, np.zeros(fs.dim, dtype=np.float32), np.zeros(fs.dim, dtype=np.float64)
            continue
        uniq, inv = np.unique(idx, return_inverse=True)
        rows = synth_rows(fs.seed, uniq, fs.dim, fs.dtype).astype(np.float64)[inv]
        yield b, k, rows.sum(axis=0).astype(np.float32), np.abs(rows).sum(axis=0)


def verify_sampled_cells(out_host: np.ndarray, first_cols: Sequence[int], cfg: ModelConfig, values, offsets, n: int,
                         seed: int = 0, features: Optional[Sequence[int]] = None) -> dict:
    """Compare `n` sampled cells of a pooled output (host array [batch, units]; feature k of `features` starts at
    column first_cols[k]) with sums of regenerated rows.  Each element is allowed the benchmark's tolerance (fp32
    tables: rel 1e-5 + abs 1e-6; fp16 tables: rel 2e-3 + abs 1e-6) plus two units in the last place of the bag's sum of
    magnitudes (2 x 2^-24 x sum |row|: what two correct fp32 summations in different orders may differ by, which
    matters for bags of a thousand rows).  Returns the cell count, the worst error as a multiple of its allowance,
    the worst plain relative error, and whether every sampled empty bag was exactly zero."""
    feats = list(range(len(cfg.features))) if features is None else list(features)
    worst, worst_rel, zeros_ok = 0.0, 0.0, True
    for b, k, expect, mags in sampled_cells(cfg, values, offsets, n, seed, features):
        fs = cfg.features[feats[k]]
        got = out_host[b, first_cols[k]:first_cols[k] + fs.dim].astype(np.float64)
        if int(offsets[k][b]) == int(offsets[k][b + 1]):
            zeros_ok = zeros_ok and bool(np.all(got == 0.0))
        rtol = 2e-3 if fs.dtype == "f16" else 1e-5
        err = np.abs(got - expect)
        allowed = rtol * np.abs(expect) + 1e-6 + 2.0 * 2.0 ** -24 * mags
        worst = max(worst, float((err / allowed).max()))
        worst_rel = max(worst_rel, float((err / np.maximum(np.abs(expect), 1e-3)).max()))
    return {"cells": n, "max_err_over_allowance": worst, "max_rel_err": worst_rel, "empty_bags_exact_zero": zeros_ok,
            "ok": bool(worst <= 1.0 and zeros_ok)}


def make_tables_numpy(cfg: ModelConfig) -> List[np.ndarray]:
    """All tables on the host (small configurations only)."""
    return [synth_table(fs.seed, fs.rows, fs.dim, fs.dtype) for fs in cfg.features]


def make_tables_device(cfg: ModelConfig, device, features: Optional[Sequence[int]] = None) -> list:
    """Tables on `device` (all of them, or only `features`), filled by the library's counter-based generator."""
    import ctypes as C

    import torch

    from . import _lib

    lib = _lib.load()
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    tables = []
    for fs in (cfg.features if features is None else [cfg.features[f] for f in features]):
        t = torch.empty((fs.rows, fs.dim), dtype=torch.float16 if fs.dtype == "f16" else torch.float32, device=dev)
        _lib.check(lib.eb_fill_table(C.c_void_p(t.data_ptr()), fs.rows, fs.dim,
                                     _lib.EB_F16 if fs.dtype == "f16" else _lib.EB_F32, fs.seed, WEIGHT_STD, idx,
                                     stream))
        tables.append(t)
    return tables
