"""GPU, benchmark-sized: cfg3 at its full size (200 fp16 tables, 120 GB, batch 16384) through size-independent
properties, since no CPU can pool 53 M rows from 120 GB of tables in test time:

* counting: with tables of ones every pooled value must equal the bag's length exactly (lengths <= 500 are exact
  in fp32) — offsets, lengths, empty bags and index handling bit-exact over the whole batch (the reference's tuner
  also measures on all-ones tables, RecFlex/tuning/measure.py:41);
* sampling: with the counter-based synthetic weights, a few thousand randomly chosen (sample, feature) outputs are
  recomputed on the CPU from regenerated rows and compared within the fp16-table tolerance;
* linearity in the schedules: two different schedule assignments give results within that tolerance everywhere.
"""
import numpy as np
import pytest
import torch

from oracle import oracle
from recflex_b200 import synth
from recflex_b200.rec_modules import FeatEmbed, Schedule

pytestmark = pytest.mark.gpu


def _enough_memory():
    if not torch.cuda.is_available():
        return False
    free, total = torch.cuda.mem_get_info(0)
    return free > 150e9


@pytest.fixture(scope="module")
def cfg3_batch():
    cfg = synth.make_config(3)
    values, offsets = synth.gen_batch(cfg, seed=42)
    pv, po = synth.pack_batch(values, offsets)
    return cfg, values, offsets, torch.from_numpy(pv).cuda(), torch.from_numpy(po).cuda()


def test_full_size_counting_with_tables_of_ones(cfg3_batch):
    if not _enough_memory():
        pytest.skip("needs about 125 GB of free device memory")
    cfg, values, offsets, dv, do = cfg3_batch
    tables = [torch.ones((fs.rows, fs.dim), dtype=torch.float16, device="cuda:0") for fs in cfg.features]
    mod = FeatEmbed("cuda:0", embed_tables=tables)
    out = mod.forward_packed(dv, do)
    mod.check_status()
    lens = torch.from_numpy(np.stack([np.diff(o) for o in offsets]).T.astype(np.float32)).cuda()  # [B, F]
    col = 0
    for f, fs in enumerate(cfg.features):
        block = out[:, col:col + fs.dim]
        assert torch.equal(block, lens[:, f:f + 1].expand(-1, fs.dim)), f"feature {f}"
        col += fs.dim
    del mod, tables, out
    torch.cuda.empty_cache()


def test_full_size_sampled_against_oracle_and_across_schedules(cfg3_batch):
    if not _enough_memory():
        pytest.skip("needs about 125 GB of free device memory")
    cfg, values, offsets, dv, do = cfg3_batch
    tables = synth.make_tables_device(cfg, "cuda:0")
    mod = FeatEmbed("cuda:0", embed_tables=tables)
    mod.set_schedules([Schedule("stream", 4) for _ in cfg.features], occupancy=6)
    out = mod.forward_packed(dv, do)
    mod.check_status()
    mod.set_schedules([Schedule("warp", 2) for _ in cfg.features], occupancy=4)
    out2 = mod.forward_packed(dv, do)
    torch.testing.assert_close(out, out2, rtol=2e-3, atol=1e-5)
    rng = np.random.default_rng(7)
    cols = np.concatenate([[0], np.cumsum([fs.dim for fs in cfg.features])])
    host = out.cpu().numpy()
    for _ in range(3000):
        f = int(rng.integers(0, len(cfg.features)))
        b = int(rng.integers(0, cfg.batch))
        fs = cfg.features[f]
        idx = values[f][offsets[f][b]:offsets[f][b + 1]].astype(np.int64)
        uniq, inv = np.unique(idx, return_inverse=True)
        if len(idx) == 0:
            expect = np.zeros(fs.dim, dtype=np.float32)
            assert np.all(host[b, cols[f]:cols[f + 1]] == 0.0)
            continue
        rows = synth.synth_rows(fs.seed, uniq, fs.dim, fs.dtype)
        expect = oracle.pool([rows], [inv], [np.array([0, len(inv)])], acc64=True)[0]
        np.testing.assert_allclose(host[b, cols[f]:cols[f + 1]], expect, rtol=2e-3, atol=1e-6)
