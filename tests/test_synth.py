"""CPU: the synthetic benchmark configurations have the shapes the benchmark definitions name."""
import numpy as np

from recflex_b200 import synth


def test_cfg1_shapes():
    cfg = synth.make_config(1)
    assert [f.dim for f in cfg.features] == [16, 16, 32, 32, 64, 64, 128, 128]
    assert all(f.rows == 100_000 and f.dtype == "f32" for f in cfg.features)
    assert cfg.batch == 256 and cfg.output_units == 480
    v, o = synth.gen_batch(cfg, 0)
    for f in range(2):
        assert np.all(np.diff(o[f]) == 1)
    for f in range(2, 8):
        d = np.diff(o[f])
        assert d.min() >= 1 and d.max() <= 20
        assert v[f].min() >= 0 and v[f].max() < 100_000


def test_cfg2_and_cfg5_share_tables():
    c2, c5 = synth.make_config(2), synth.make_config(5)
    assert len(c2.features) == 50 and c2.batch == 4096 and c5.batch == 16384
    assert [(f.rows, f.dim, f.seed) for f in c2.features] == [(f.rows, f.dim, f.seed) for f in c5.features]
    assert sum(f.length == "onehot" for f in c2.features) == 20
    assert sum(f.length == "empty" for f in c5.features) == 5
    assert sum(f.index == "uniform" for f in c5.features) == 20
    assert all(1e3 <= f.rows <= 1e7 and f.dim in (4, 8, 16, 32, 64, 128) for f in c2.features)


def test_cfg3_size_and_lengths():
    cfg = synth.make_config(3)
    assert len(cfg.features) == 200 and cfg.batch == 16384
    assert abs(cfg.table_bytes - 120e9) < 1e9
    assert all(f.dtype == "f16" and f.dim in (8, 16, 32, 64, 128, 256) for f in cfg.features)
    v, o = synth.gen_feature_batch(cfg.features[0], 16384, 0)
    lens = np.diff(o)
    assert lens.max() <= 500 and 0.03 < (lens == 0).mean() < 0.07
    assert v.min() >= 0 and v.max() < cfg.features[0].rows


def test_cfg4_shape():
    cfg = synth.make_config(4)
    assert len(cfg.features) == 400 and cfg.batch == 65536
    assert sum(f.rows == 100_000_000 and f.dim == 64 for f in cfg.features) == 40
    assert cfg.table_bytes > 500e9


def test_batches_are_seeded_and_bytes_formula():
    cfg = synth.make_config(2, row_scale=0.01, batch=64)
    a = synth.gen_batch(cfg, 3)
    b = synth.gen_batch(cfg, 3)
    c = synth.gen_batch(cfg, 4)
    assert all(np.array_equal(x, y) for x, y in zip(a[0], b[0]))
    assert any(not np.array_equal(x, y) for x, y in zip(a[0], c[0]))
    expect = sum(int(o[-1]) * f.row_bytes + int(o[-1]) * 4 + 65 * 4 for f, o in zip(cfg.features, a[1]))
    assert synth.algorithmic_bytes(cfg, a[1], 4) == expect
    pv, po = synth.pack_batch(*a)
    assert po.shape == (50, 65) and len(pv) == sum(len(x) for x in a[0])


def test_retune_trigger_is_bucketed():
    from recflex_b200.tuning import InputStats, needs_retune

    old = [InputStats(10.0, 40, 0.0), InputStats(1.0, 1, 0.0), InputStats(3.0, 9, 0.1)]
    new = [InputStats(11.0, 44, 0.0), InputStats(10.0, 30, 0.0), InputStats(3.1, 9, 0.2)]
    assert needs_retune(old, new) == [1]
