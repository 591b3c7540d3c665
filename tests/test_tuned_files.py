"""Host-side checks of the tuner's persisted results (no GPU): the JSON round trip and the committed schedule files."""
import glob
import json
import os

from recflex_b200 import _lib, synth
from recflex_b200.rec_modules import Schedule
from recflex_b200.tuning import InputStats, TuneResult

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_tune_result_round_trip(tmp_path):
    res = TuneResult([Schedule("warp", 4), Schedule("pipe", 8, 64)], 5, {}, {4: 1.5, 5: 1.25},
                     [InputStats(700.0, 880, 0.0), InputStats(1.0, 1, 0.0)], overlap=1)
    path = os.path.join(tmp_path, "t.json")
    res.save(path, workload="x")
    back = TuneResult.load(path)
    assert back.schedules == res.schedules and back.occupancy == 5 and back.overlap == 1
    assert back.global_ms == res.global_ms and back.stats[0].max_len == 880
    with open(path) as f:
        assert json.load(f)["workload"] == "x"


def test_result_files_without_an_overlap_entry_load_as_serial(tmp_path):
    path = os.path.join(tmp_path, "old.json")
    with open(path, "w") as f:
        json.dump({"occupancy": 3, "schedules": [{"kind": "pipe", "unroll": 8, "bags_per_tile": 0}]}, f)
    assert TuneResult.load(path).overlap == 0


def test_committed_schedule_files_fit_their_workloads():
    files = sorted(glob.glob(os.path.join(ROOT, "recflex_b200", "tuned", "cfg*.json")))
    assert files
    for path in files:
        cfg_id = int(os.path.basename(path)[3:-5])
        res = TuneResult.load(path)
        assert len(res.schedules) == len(synth.make_config(cfg_id, row_scale=1e-4).features)
        assert 1 <= res.occupancy <= 8 and 0 <= res.overlap <= res.occupancy
        for s in res.schedules:
            assert s.kind in _lib.SCHED_NAMES and s.unroll in (1, 2, 4, 6, 8)
            assert s.bags_per_tile == 0 or (s.bags_per_tile & (s.bags_per_tile - 1)) == 0
