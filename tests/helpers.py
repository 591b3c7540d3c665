"""Shared helpers of the GPU parity tests."""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle
from recflex_b200 import synth
from recflex_b200.rec_modules import FeatEmbed, Schedule

# tolerances of the benchmark definition: fp32 tables rel 1e-5 / abs 1e-6,
# fp16 tables (fp32 accumulation) rel 2e-3
TOL = {"f32": dict(rtol=1e-5, atol=1e-6), "f16": dict(rtol=2e-3, atol=1e-6)}


def device_tables(tables_np, device="cuda:0"):
    return [torch.from_numpy(t).to(device) for t in tables_np]


def to_device(arrs, device="cuda:0", dtype=None):
    return [torch.from_numpy(np.ascontiguousarray(a if dtype is None else a.astype(dtype))).to(device) for a in arrs]


def check_against_oracle(out: torch.Tensor, tables_np, values, offsets, dtype_tag: str):
    """Compare with the float64-accumulating oracle; empty bags must be exactly zero."""
    expect = oracle.pool(tables_np, values, offsets, acc64=True)
    got = out.detach().cpu().numpy()
    assert got.shape == expect.shape
    np.testing.assert_allclose(got, expect, **TOL[dtype_tag])
    col = 0
    for t, o in zip(tables_np, offsets):
        o = np.asarray(o)
        empty = np.nonzero(o[1:] == o[:-1])[0]
        if len(empty):
            assert np.all(got[empty, col:col + t.shape[1]] == 0.0), "empty bags must pool to exactly 0"
        col += t.shape[1]


def all_schedules(kind: str, unroll: int, n: int, bags_per_tile: int = 0):
    return [Schedule(kind, unroll, bags_per_tile) for _ in range(n)]


def small_model(cfg_id: int, row_scale: float, batch: int, seed: int = 0):
    cfg = synth.make_config(cfg_id, row_scale=row_scale, batch=batch)
    tables = synth.make_tables_numpy(cfg)
    values, offsets = synth.gen_batch(cfg, seed)
    return cfg, tables, values, offsets


def compacted_model(cfg, values):
    """Tables too large for the host: keep only the rows a batch touches (regenerated from the counter-based
    weights) and renumber the indices.  Returns (tables, values) for the oracle; offsets stay as they are."""
    from concurrent.futures import ThreadPoolExecutor

    def one(args):
        fs, v = args
        uniq, inv = np.unique(np.asarray(v, dtype=np.int64), return_inverse=True)
        if len(uniq) == 0:
            uniq = np.zeros(1, dtype=np.int64)
        return synth.synth_rows(fs.seed, uniq, fs.dim, fs.dtype), inv.astype(np.int64)

    with ThreadPoolExecutor(max_workers=16) as pool:
        res = list(pool.map(one, zip(cfg.features, values)))
    return [r[0] for r in res], [r[1] for r in res]
