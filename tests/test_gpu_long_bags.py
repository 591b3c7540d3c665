"""GPU: bags far longer than the rest (the block-per-bag case; reference: mbs::SparseSegmentReduceCore,
examples/csrc/include/multi_block_per_sample_kernel.cuh:17-112, which splits long bags over blocks and adds the
parts with atomics).  Here the warp that meets such a bag hands it to eb_longbag_kernel, where many warps pool
segments of it and the last one adds the partial sums in order."""
import time

import numpy as np
import pytest
import torch

from oracle import oracle
from recflex_b200.rec_modules import FeatEmbed, Schedule
from tests.helpers import TOL

pytestmark = pytest.mark.gpu


def _model(batch, long_at, long_len, seed=0):
    """Three features over small tables; every bag has 0 to 5 entries except the ones at `long_at`."""
    rng = np.random.default_rng(seed)
    specs = [(60000, 256, np.float16), (40000, 64, np.float16), (50000, 32, np.float32)]
    tables = [(rng.standard_normal((r, d)) * 0.01).astype(t) for r, d, t in specs]
    values, offsets = [], []
    for f, (r, d, t) in enumerate(specs):
        lens = rng.integers(0, 6, batch)
        for i, b in enumerate(long_at):
            if (i + f) % 3 != 2:  # not every feature is long at every position
                lens[b] = long_len + 17 * i + f
        o = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        offsets.append(o)
        values.append(rng.integers(0, r, o[-1]).astype(np.int32))
    return tables, values, offsets


def _check(out, tables, values, offsets):
    expect = oracle.pool(tables, values, offsets, acc64=True)
    mags = oracle.pool([np.abs(t) for t in tables], values, offsets, acc64=True)
    got = out.float().cpu().numpy()
    col = 0
    for t in tables:  # fp32 sums of 1e5 terms in another order: allow the summation-order slack on top
        tol = TOL["f16" if t.dtype == np.float16 else "f32"]
        w = slice(col, col + t.shape[1])
        bound = tol["rtol"] * np.abs(expect[:, w]) + tol["atol"] + 4.0 * 2.0 ** -24 * mags[:, w]
        assert (np.abs(got[:, w] - expect[:, w]) <= bound).all()
        col += t.shape[1]


@pytest.mark.parametrize("kind", ["stream", "pipe"])
def test_long_bags_are_handed_over_and_match_the_oracle(kind):
    batch = 2048
    long_at = [0, 37, 38, 1000, 1023, 1024, 2047]  # first bag, neighbours, around a tile edge, last bag
    tables, values, offsets = _model(batch, long_at, 150_000)
    mod = FeatEmbed("cuda:0", embed_tables=[torch.from_numpy(t).cuda() for t in tables])
    mod.set_schedules([Schedule(kind, 4) for _ in tables], occupancy=4)
    dv = [torch.from_numpy(v).cuda() for v in values]
    do = [torch.from_numpy(o).cuda() for o in offsets]

    def timed():
        for _ in range(2):
            out = mod(dv, do)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(5):
            out = mod(dv, do)
        torch.cuda.synchronize()
        return out, (time.perf_counter() - t0) / 5 * 1e3

    out, split_ms = timed()
    mod.check_status()
    _check(out, tables, values, offsets)
    mod.set_long_bag_split(0)  # every bag pooled by the warp that meets it
    ref, inplace_ms = timed()
    _check(ref, tables, values, offsets)
    print(f"\\n{kind}: long bags handed over {split_ms:.3f} ms, pooled in place {inplace_ms:.3f} ms per forward")
    assert split_ms < inplace_ms, "handing the long bags to many warps must beat one warp per bag"
    # two runs give the same bits: the partial sums are added in segment order, not as they arrive
    mod.set_long_bag_split(1 << 20)
    assert torch.equal(mod(dv, do), out)


def test_more_long_bags_than_the_list_holds_and_narrow_output():
    batch = 1024
    tables, values, offsets = _model(batch, list(range(0, 1024, 3)), 3000, seed=1)  # 342 positions, list holds 256
    mod = FeatEmbed("cuda:0", embed_tables=[torch.from_numpy(t).cuda() for t in tables])
    mod.set_long_bag_split(64 * 1024)  # 3000 rows of 64 bytes and more count as long here
    dv = [torch.from_numpy(v).cuda() for v in values]
    do = [torch.from_numpy(o).cuda() for o in offsets]
    out = mod(dv, do)
    mod.check_status()
    _check(out, tables, values, offsets)
    mod.set_output_dtype(torch.bfloat16)
    narrow = mod(dv, do)
    mags = torch.from_numpy(oracle.pool([np.abs(t) for t in tables], values, offsets, acc64=True)).cuda()
    assert ((narrow.float() - out).abs() <= 2 * 2.0 ** -8 * mags + 1e-7).all()


def test_long_bags_in_peer_mode_and_packed_input():
    from recflex_b200 import synth

    world, rows = 4, 256
    tables, values, offsets = _model(world * rows, [5, 300, 1023], 120_000, seed=2)
    mod = FeatEmbed("cuda:0", embed_tables=[torch.from_numpy(t).cuda() for t in tables])
    units = mod.output_units
    outs = [torch.full((rows, units), float("nan"), device="cuda:0") for _ in range(world)]
    mod.forward_peers([torch.from_numpy(v).cuda() for v in values], [torch.from_numpy(o).cuda() for o in offsets],
                      [o.data_ptr() for o in outs], units)
    torch.cuda.synchronize()
    _check(torch.cat(outs), tables, values, offsets)
    pv, po = synth.pack_batch(values, offsets)
    _check(mod.forward_packed(torch.from_numpy(pv).cuda(), torch.from_numpy(po).cuda()), tables, values, offsets)
