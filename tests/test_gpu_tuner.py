"""GPU: the two-stage tuner picks schedules, keeps parity, round-trips through JSON."""
import os

import pytest
import torch

from recflex_b200.rec_modules import FeatEmbed, Schedule
from recflex_b200.tuning import TuneConfig, Tuner, TuneResult
from tests.helpers import check_against_oracle, device_tables, small_model, to_device

pytestmark = pytest.mark.gpu


def test_tuner_end_to_end(tmp_path):
    cfg, tables, values, offsets = small_model(2, 0.02, 2048)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    dv, do = to_device(values), to_device(offsets)
    tc = TuneConfig(occupancies=(4, 8), reps=1, global_reps=2, min_replicas=16)
    tuner = Tuner(mod, [(dv, do)], tc)
    assert len(tuner.clusters()) < len(tables)  # look-alike features share one representative
    res = tuner.tune()
    assert res.occupancy in (4, 8) and len(res.schedules) == len(tables)
    assert set(res.global_ms) == {4, 8} and all(v > 0 for v in res.global_ms.values())
    # local stage measured every candidate of every feature at every occupancy
    for f in range(len(tables)):
        for occ in (4, 8):
            assert len(res.local_times[f][occ]) == len(tuner._cands[f])
            assert all(t > 0 for t in res.local_times[f][occ])
    # the tuned module still computes the right thing
    got, occ = mod.get_schedules()
    assert occ == res.occupancy and got == res.schedules
    out = mod(dv, do)
    mod.check_status()
    check_against_oracle(out, tables, values, offsets, "f32")
    # persistence
    path = os.path.join(tmp_path, "tuned.json")
    res.save(path, workload=cfg.name)
    back = TuneResult.load(path)
    assert back.schedules == res.schedules and back.occupancy == res.occupancy and back.overlap == res.overlap
    assert 0 <= res.overlap <= res.occupancy
    # one-hot features never get a multi-row unroll from the slot-per-bag candidates
    onehot = [f for f, fs in enumerate(cfg.features) if fs.length == "onehot"]
    for f in onehot:
        assert all(not (c.kind == 1 and c.unroll > 1) for c in tuner.candidates(f))
    # mutation validation: every mutation is timed, the pick is one of them
    times, pick = tuner.mutation_validation(res, onehot[0])
    assert len(times) == len(tuner.candidates(onehot[0])) and all(t > 0 for t in times)


def test_naive_tuning_and_retune():
    cfg, tables, values, offsets = small_model(2, 0.02, 512)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables[:6]))
    dv, do = to_device(values[:6]), to_device(offsets[:6])
    tc = TuneConfig(occupancies=(4,), reps=1, global_reps=1, kinds=("warp", "stream"), unrolls=(2, 4))
    tuner = Tuner(mod, [(dv, do)], tc)
    res = tuner.tune_naive(occupancy=4)
    assert len(res.schedules) == 6
    res = tuner.tune()
    # shifted inputs: feature 0's bags become 8x longer -> only that feature is re-tuned
    v0 = torch.cat([dv[0]] * 8)
    o0 = do[0] * 8
    shifted = ([v0] + dv[1:], [o0] + do[1:])
    res2 = tuner.retune(res, [shifted])
    assert list(res2.local_times) == [0]
    out = mod(*shifted)
    mod.check_status()
    # the retuned module on the shifted batch against the oracle
    import numpy as np

    sv = [np.concatenate([values[0]] * 8)] + list(values[1:6])
    so = [offsets[0] * 8] + list(offsets[1:6])
    check_against_oracle(out, tables[:6], sv, so, "f32")


def test_schedule_config_restricts_candidates_and_fixed_thread_binding(tmp_path):
    """A reference schedule_config.txt names each feature's candidate classes (RecFlex/parser.py:19-26); the tuner
    must pick only among them.  Then the fixed-thread-binding ablation (RecFlex/tuning/tuner.py:312-357)."""
    from recflex_b200 import _lib
    from recflex_b200.parser import parse_schedule_types

    cfg, tables, values, offsets = small_model(2, 0.02, 1024)
    tables, values, offsets = tables[:8], values[:8], offsets[:8]
    lines = ["OneHotSchedule,WarpPerSampleSchedule", "ReduceByKeySchedule", "MultiBlockPerSampleSchedule,NoSuchSchedule",
             "OneBlockMultiSampleSchedule", "WarpPerSampleSchedule", "ReduceByKeySchedule,MultiBlockPerSampleSchedule",
             "OneHotMultiBlockSchedule", "MultiBlockPerSampleSchedule"]
    path = os.path.join(tmp_path, "schedule_config.txt")
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    allowed = parse_schedule_types(path)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    dv, do = to_device(values), to_device(offsets)
    tc = TuneConfig(occupancies=(4,), reps=1, global_reps=1, uniform_portfolio=(), hybrid_min_len=(), refine_top=0)
    tuner = Tuner(mod, [(dv, do)], tc, candidates_from=allowed)
    res = tuner.tune()
    for f, s in enumerate(res.schedules):
        names = {k for k in allowed[f] if k is not None}
        assert _lib.SCHED_NAMES[s.kind] in names, (f, s, names)
    check_against_oracle(mod(dv, do), tables, values, offsets, "f32")
    fixed, fixed_ms, dyn_ms = tuner.tune_fixed_thread_binding(res, "max")
    assert len(fixed) == 8 and all(n >= 1 and n & (n - 1) == 0 for n in fixed) and fixed_ms > 0 and dyn_ms > 0
    got, _ = mod.get_schedules()
    assert all(s.bags_per_tile == 0 for s in got)  # the run-time binding is back
    pinned = [Schedule(s.kind, s.unroll, fixed[f]) for f, s in enumerate(res.schedules)]
    mod.set_schedules(pinned, occupancy=res.occupancy)
    check_against_oracle(mod(dv, do), tables, values, offsets, "f32")
