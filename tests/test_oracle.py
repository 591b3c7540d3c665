"""CPU: the oracle against the golden fixtures produced from the reference (tests/golden/make_golden.py)."""
import json
import os

import numpy as np
import pytest

from oracle import oracle
from recflex_b200 import synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = ["mixed_f32", "long_f32", "onehot_f32", "mixed_f16"]


def load_case(name):
    z = np.load(os.path.join(GOLD, "pool_golden.npz"))
    raw = [str(s).split("\n") for s in z[f"{name}.raw"]]
    batch = int(z[f"{name}.batch"])
    raw = [lines if len(lines) == batch else lines + [""] * (batch - len(lines)) for lines in raw]
    tables = []
    i = 0
    while f"{name}.table{i}" in z:
        tables.append(z[f"{name}.table{i}"])
        i += 1
    return tables, raw, z[f"{name}.expect"]


@pytest.mark.parametrize("name", CASES)
def test_pool_matches_reference_formula(name):
    tables, raw, expect = load_case(name)
    parsed = [oracle.parse_bags(lines) for lines in raw]
    values = [p[0] for p in parsed]
    offsets = [p[1] for p in parsed]
    # the reference's own check uses atol = rtol = 1e-4 (examples/test.py:85); the benchmark's fp32 tolerance
    # (rel 1e-5 / abs 1e-6) covers the summation-order difference between torch's sum and a serial sum
    for acc64 in (False, True):
        got = oracle.pool(tables, values, offsets, acc64=acc64)
        np.testing.assert_allclose(got, expect, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(oracle.pool_numpy(tables, values, offsets), expect, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(oracle.pool_torch(tables, values, offsets).numpy(), expect, rtol=1e-5, atol=1e-6)
    # empty lines pool to exactly zero
    col = 0
    for t, o in zip(tables, offsets):
        empty = np.nonzero(o[1:] == o[:-1])[0]
        assert np.all(oracle.pool(tables, values, offsets)[empty, col:col + t.shape[1]] == 0.0)
        col += t.shape[1]


def test_parser_matches_reference_host_parser():
    with open(os.path.join(GOLD, "parse_golden.json")) as f:
        gold = json.load(f)
    for case in gold["ws"]:
        v, o = oracle.parse_bags(case["lines"])
        assert v.tolist() == case["indices"]
        assert o.tolist() == case["segment_offsets"]
        # reference tiling for the ws schedule: one tile (= block) per `tile_size` bags
        assert case["num_tiles"] == -(-len(case["lines"]) // case["tile_size"]) == case["num_blocks"]
    oh = gold["onehot"]
    v, o = oracle.parse_bags(oh["lines"])
    assert v.tolist() == oh["indices"] and o.tolist() == list(range(len(oh["lines"]) + 1))


def test_library_parser_matches_reference_host_parser(lib):
    from recflex_b200.rec_modules import parse_bags

    with open(os.path.join(GOLD, "parse_golden.json")) as f:
        gold = json.load(f)
    for case in gold["ws"]:
        v, o = parse_bags(case["lines"])
        assert v.tolist() == case["indices"]
        assert o.tolist() == case["segment_offsets"]


def test_synthetic_weights_agree_between_c_and_numpy():
    ids = np.array([0, 1, 2, 999, 12345678, 49_999_999], dtype=np.int64)
    for seed, dim in ((1003000, 8), (1003017, 256), (7, 33)):
        a = oracle.synth_rows(seed, ids, dim)
        b = synth.synth_rows(seed, ids, dim, "f32")
        assert np.array_equal(a, b)
    t = synth.synth_table(5, 20000, 16, "f32")
    assert abs(float(t.std()) - synth.WEIGHT_STD) < 2e-4 and abs(float(t.mean())) < 2e-4


def test_oracle_rejects_out_of_range_index():
    t = [np.ones((4, 4), dtype=np.float32)]
    with pytest.raises(ValueError):
        oracle.pool(t, [np.array([0, 4])], [np.array([0, 2])])
    out = oracle.pool(t, [np.array([0, 4])], [np.array([0, 2])], strict=False)
    assert np.all(out == 1.0)


def test_text_format_readers_match_the_reference(tmp_path):
    from recflex_b200 import parser

    with open(os.path.join(GOLD, "parse_golden.json")) as f:
        gold = json.load(f)["formats"]
    for name, text in gold["files"].items():
        (tmp_path / name).write_text(text)
    fnames = [str(tmp_path / f"f{i}.txt") for i in range(3)]
    assert [list(t) for t in parser.parse_table_shapes(str(tmp_path / "table_config.txt"))] == gold["table_shapes"]
    assert parser.parse_raw_data_batches(str(tmp_path / "batch_sizes.txt"), fnames, 4, seed=3) == gold["feat_major"]
    assert parser.parse_raw_data_batches(str(tmp_path / "batch_sizes.txt"), fnames, 4, seed=3,
                                         feat_major=False) == gold["batch_major"]
    (tmp_path / "schedule_config.txt").write_text("OneHotSchedule,OneHotMultiBlockSchedule\nWarpPerSampleSchedule,ReduceByKeySchedule,Nope\n")
    assert parser.parse_schedule_types(str(tmp_path / "schedule_config.txt")) == [["group", "group"], ["group", "flat", None]]
