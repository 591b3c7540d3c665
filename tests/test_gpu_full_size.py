"""GPU, benchmark-sized: the configurations the benchmark times, at their full size and WITH the tuned schedule
assignments the benchmark loads (recflex_b200/tuned/*.json: schedules, occupancy and kernel overlap).

cfg3 (200 fp16 tables, 120 GB, batch 16384) cannot be pooled on a CPU in test time, so it is checked through
size-independent properties:

* counting: with tables of ones every pooled value must equal the bag's length exactly (lengths <= 500 are exact
  in fp32) — offsets, lengths, empty bags and index handling bit-exact over the whole batch (the reference's tuner
  also measures on all-ones tables, RecFlex/tuning/measure.py:41);
* sampling: with the counter-based synthetic weights, a few thousand randomly chosen (sample, feature) outputs are
  recomputed on the CPU from regenerated rows and compared within the fp16-table tolerance
  (the definition of the expected value is the reference checker's, examples/test.py:68-86);
* agreement between different schedule assignments within that tolerance everywhere.

cfg2 and cfg5 (fp32, 8.7 GB of tables) are compared with the oracle over the WHOLE batch: the oracle gets the
rows the batch touches, regenerated on the host.
"""
import numpy as np
import pytest
import torch

from oracle import oracle
from recflex_b200 import synth
from recflex_b200.rec_modules import FeatEmbed, Schedule
from recflex_b200.tuning import TuneResult, tuned_path
from tests.helpers import check_against_oracle, compacted_model

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


def _assignments(cfg):
    """name -> function that installs the assignment on a module; the benchmark's own comes first."""
    tuned = TuneResult.load(tuned_path("cfg3"))
    assert len(tuned.schedules) == len(cfg.features)
    assert any(s.kind == 5 for s in tuned.schedules), "the benchmarked cfg3 assignment uses the pipelined schedule"

    def uniform(kind, unroll, occ):
        def install(mod):
            mod.set_kernel_overlap(0)
            mod.set_schedules([Schedule(kind, unroll) for _ in cfg.features], occupancy=occ)
        return install

    return {"tuned": tuned.apply, "stream-u4-occ6": uniform("stream", 4, 6), "warp-u2-occ4": uniform("warp", 2, 4)}


def test_full_size_counting_with_tables_of_ones(cfg3_batch):
    if not _enough_memory():
        pytest.skip("needs about 125 GB of free device memory")
    cfg, values, offsets, dv, do = cfg3_batch
    tables = [torch.ones((fs.rows, fs.dim), dtype=torch.float16, device="cuda:0") for fs in cfg.features]
    mod = FeatEmbed("cuda:0", embed_tables=tables)
    lens = torch.from_numpy(np.stack([np.diff(o) for o in offsets]).T.astype(np.float32)).cuda()  # [B, F]
    installers = _assignments(cfg)
    for name in ("tuned", "stream-u4-occ6"):
        installers[name](mod)
        out = mod.forward_packed(dv, do)
        mod.check_status()
        col = 0
        for f, fs in enumerate(cfg.features):
            block = out[:, col:col + fs.dim]
            assert torch.equal(block, lens[:, f:f + 1].expand(-1, fs.dim)), f"{name}: feature {f}"
            col += fs.dim
        del out
    del mod, tables
    torch.cuda.empty_cache()


def test_full_size_sampled_against_oracle_and_across_schedules(cfg3_batch):
    if not _enough_memory():
        pytest.skip("needs about 125 GB of free device memory")
    cfg, values, offsets, dv, do = cfg3_batch
    tables = synth.make_tables_device(cfg, "cuda:0")
    mod = FeatEmbed("cuda:0", embed_tables=tables)
    installers = _assignments(cfg)
    installers["tuned"](mod)  # exactly what bench.py times
    out = mod.forward_packed(dv, do)
    mod.check_status()
    for name in ("stream-u4-occ6", "warp-u2-occ4"):
        installers[name](mod)
        other = mod.forward_packed(dv, do)
        mod.check_status()
        torch.testing.assert_close(out, other, rtol=2e-3, atol=1e-5, msg=lambda m: f"tuned vs {name}: {m}")
        del other
    cols = np.concatenate([[0], np.cumsum([fs.dim for fs in cfg.features])])
    host = out.cpu().numpy()
    for b, f, expect64, _ in synth.sampled_cells(cfg, values, offsets, 3000, seed=7):
        fs = cfg.features[f]
        got = host[b, cols[f]:cols[f + 1]]
        idx = values[f][offsets[f][b]:offsets[f][b + 1]].astype(np.int64)
        if len(idx) == 0:
            assert np.all(got == 0.0)
            continue
        uniq, inv = np.unique(idx, return_inverse=True)
        rows = synth.synth_rows(fs.seed, uniq, fs.dim, fs.dtype)
        expect = oracle.pool([rows], [inv], [np.array([0, len(inv)])], acc64=True)[0]
        np.testing.assert_allclose(got, expect, rtol=2e-3, atol=1e-6)
        np.testing.assert_allclose(expect64, expect, rtol=1e-6, atol=1e-7)  # the benchmark's self-check agrees with the oracle
    del mod, tables, out
    torch.cuda.empty_cache()


@pytest.mark.parametrize("workload", ["cfg2", "cfg5"])
def test_full_size_fp32_configs_with_tuned_schedules_against_oracle(workload):
    if not torch.cuda.is_available() or torch.cuda.mem_get_info(0)[0] < 16e9:
        pytest.skip("needs about 12 GB of free device memory")
    cfg = synth.make_config(int(workload[3:]))
    values, offsets = synth.gen_batch(cfg, seed=42)
    tables = synth.make_tables_device(cfg, "cuda:0")
    mod = FeatEmbed("cuda:0", embed_tables=tables)
    tuned = TuneResult.load(tuned_path(workload))
    assert len(tuned.schedules) == len(cfg.features)
    tuned.apply(mod)
    dv = [torch.from_numpy(v).cuda() for v in values]
    do = [torch.from_numpy(o).cuda() for o in offsets]
    out = mod(dv, do)
    mod.check_status()
    small_tables, small_values = compacted_model(cfg, values)
    if workload == "cfg2":
        check_against_oracle(out, small_tables, small_values, offsets, "f32")
        return
    # cfg5 stretches bags to a thousand entries and more.  Over 31 M cells two correct fp32 summations in different
    # orders can differ by more than abs 1e-6, so each cell gets, on top of rel 1e-5 / abs 1e-6, an allowance for
    # the order of summation: 2 ulp-fractions (2 x 2^-24) of the bag's sum of magnitudes.
    expect = oracle.pool(small_tables, small_values, offsets, acc64=True)
    mags = oracle.pool([np.abs(t) for t in small_tables], small_values, offsets, acc64=True)
    got = out.cpu().numpy()
    tol = 1e-5 * np.abs(expect) + 1e-6 + 2.0 * 2.0 ** -24 * mags
    bad = np.abs(got - expect) > tol
    assert not bad.any(), f"{int(bad.sum())} cells out of tolerance, worst {float(np.abs(got - expect).max()):.3e}"
    col = 0
    for fs, o in zip(cfg.features, offsets):
        empty = np.nonzero(np.diff(o) == 0)[0]
        assert np.all(got[empty, col:col + fs.dim] == 0.0), "empty bags must pool to exactly 0"
        col += fs.dim
