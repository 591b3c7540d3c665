"""GPU parity: the fused CUDA forward (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle
from recflex_b200 import synth
from recflex_b200.rec_modules import FeatEmbed, Schedule
from tests.helpers import (TOL, all_schedules, check_against_oracle, device_tables, small_model, to_device)

pytestmark = pytest.mark.gpu

KINDS = ["group", "warp", "flat", "stream", "pipe"]
UNROLLS = [1, 2, 4, 8]


@pytest.fixture(scope="module")
def cfg1():
    cfg, tables, values, offsets = small_model(1, 1.0, 256)
    return cfg, tables, values, offsets, FeatEmbed("cuda:0", embed_tables=device_tables(tables))


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("unroll", UNROLLS)
def test_cfg1_every_schedule(cfg1, kind, unroll):
    cfg, tables, values, offsets, mod = cfg1
    mod.set_schedules(all_schedules(kind, unroll, len(tables)), occupancy=4)
    out = mod(to_device(values), to_device(offsets))
    mod.check_status()
    check_against_oracle(out, tables, values, offsets, "f32")


@pytest.mark.parametrize("cfg_id,scale,batch,tag", [(3, 2e-4, 700, "f16"), (2, 0.01, 515, "f32"), (5, 0.01, 300, "f32")])
def test_pipe_with_six_rows_per_macro_step(cfg_id, scale, batch, tag):
    """The 48 KB ring of the pipelined schedule (unroll 6, two macro-steps deep): the one unroll that is not a power
    of two; and only the pipelined schedule takes it."""
    from recflex_b200._lib import EbError

    cfg, tables, values, offsets = small_model(cfg_id, scale, batch)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    dv, do = to_device(values), to_device(offsets)
    for occ in (3, 4):
        mod.set_schedules(all_schedules("pipe", 6, len(tables)), occupancy=occ)
        out = mod(dv, do)
        mod.check_status()
        check_against_oracle(out, tables, values, offsets, tag)
    mixed = [Schedule("pipe", 6) if f % 2 else Schedule("stream", 4) for f in range(len(tables))]
    mod.set_schedules(mixed, occupancy=4)  # the kernel with every schedule
    check_against_oracle(mod(dv, do), tables, values, offsets, tag)
    with pytest.raises(EbError):
        mod.set_schedules(all_schedules("stream", 6, len(tables)))


@pytest.mark.parametrize("occupancy", [1, 2, 3, 4, 5, 6, 7, 8])
def test_cfg1_every_occupancy(cfg1, occupancy):
    cfg, tables, values, offsets, mod = cfg1
    mod.set_schedules(all_schedules("flat", 4, len(tables)), occupancy=occupancy)
    assert mod.max_concurrent_blocks == occupancy * torch.cuda.get_device_properties(0).multi_processor_count
    out = mod(to_device(values), to_device(offsets))
    check_against_oracle(out, tables, values, offsets, "f32")


def test_cfg1_matches_torch_embedding_bag(cfg1):
    cfg, tables, values, offsets, mod = cfg1
    mod.set_schedules(all_schedules("auto", 0, len(tables)), occupancy=4)
    out = mod(to_device(values), to_device(offsets)).cpu()
    ref = oracle.pool_torch(tables, values, offsets)
    torch.testing.assert_close(out, ref, **TOL["f32"])


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("cfg_id,scale,batch,tag", [(2, 0.01, 1000, "f32"), (3, 2e-4, 777, "f16"), (5, 0.01, 600, "f32"),
                                                    (4, 1e-4, 300, "f16")])
def test_scaled_configs(kind, cfg_id, scale, batch, tag):
    cfg, tables, values, offsets = small_model(cfg_id, scale, batch)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    for unroll in (2, 8):
        mod.set_schedules(all_schedules(kind, unroll, len(tables)))
        out = mod(to_device(values), to_device(offsets))
        mod.check_status()
        check_against_oracle(out, tables, values, offsets, tag)


def test_int64_indices_and_offsets_without_end(cfg1):
    cfg, tables, values, offsets, mod = cfg1
    mod.set_schedules(all_schedules("flat", 4, len(tables)))
    v64 = to_device(values, dtype=np.int64)
    o64 = to_device(offsets, dtype=np.int64)
    out = mod(v64, o64)
    check_against_oracle(out, tables, values, offsets, "f32")
    out2 = mod(v64, [o[:-1].contiguous() for o in o64], include_last_offset=False)
    assert torch.equal(out, out2)
    out3 = mod(to_device(values), [o[:-1].contiguous() for o in to_device(offsets)], include_last_offset=False)
    assert torch.equal(out, out3)


def test_packed_and_host_paths(cfg1):
    cfg, tables, values, offsets, mod = cfg1
    mod.set_schedules(all_schedules("flat", 4, len(tables)))
    ref = mod(to_device(values), to_device(offsets))
    pv, po = synth.pack_batch(values, offsets)
    out = mod.forward_packed(torch.from_numpy(pv).cuda(), torch.from_numpy(po).cuda())
    assert torch.equal(out, ref)
    hv = torch.from_numpy(pv).pin_memory()
    ho = torch.from_numpy(po).pin_memory()
    hout = mod.forward_host(hv, ho)
    torch.cuda.synchronize()
    assert torch.equal(hout, ref.cpu())


@pytest.mark.parametrize("kind", KINDS)
def test_ragged_edges(kind):
    """Empty bags, all-empty features, one giant bag, batch sizes around the 32-bag chunk."""
    rng = np.random.default_rng(5)
    dims = [4, 8, 12, 20, 32, 64, 128, 256, 3, 7, 100]
    dts = [np.float32, np.float16]
    for batch in (1, 31, 32, 33, 95):
        tables, values, offsets = [], [], []
        for i, d in enumerate(dims):
            rows = 50 + 13 * i
            tables.append((rng.standard_normal((rows, d)) * 0.1).astype(dts[i % 2]))
            mode = i % 4
            if mode == 0:
                lens = rng.integers(0, 3, batch)
            elif mode == 1:
                lens = np.zeros(batch, dtype=np.int64)
            elif mode == 2:
                lens = np.zeros(batch, dtype=np.int64)
                lens[batch // 2] = 700
            else:
                lens = rng.integers(0, 70, batch)
            o = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
            offsets.append(o)
            values.append(rng.integers(0, rows, o[-1]).astype(np.int32))
        mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
        for unroll in (1, 4):
            mod.set_schedules(all_schedules(kind, unroll, len(dims)))
            out = mod(to_device(values), to_device(offsets))
            mod.check_status()
            expect = oracle.pool(tables, values, offsets, acc64=True)
            np.testing.assert_allclose(out.cpu().numpy(), expect, rtol=2e-3, atol=1e-5)


def test_output_slice_with_wider_leading_dimension(cfg1):
    cfg, tables, values, offsets, mod = cfg1
    mod.set_schedules(all_schedules("flat", 4, len(tables)))
    ref = mod(to_device(values), to_device(offsets))
    wide = torch.full((ref.shape[0], ref.shape[1] + 37), -7.0, device="cuda:0")
    out = mod(to_device(values), to_device(offsets), out=wide)
    assert torch.equal(out[:, : ref.shape[1]], ref)
    assert torch.all(out[:, ref.shape[1]:] == -7.0)


def test_bad_inputs_are_flagged_not_dereferenced(cfg1):
    cfg, tables, values, offsets, mod = cfg1
    from recflex_b200._lib import EbError

    mod.set_schedules(all_schedules("flat", 4, len(tables)))
    bad = [v.copy() for v in values]
    bad[3][5] = tables[3].shape[0] + 12345  # far outside the table
    bad[4][0] = -1
    out = mod(to_device(bad), to_device(offsets))
    with pytest.raises(EbError):
        mod.check_status()
    # the rest of the output is still right: rows with a bad index miss only that term
    good = mod(to_device(values), to_device(offsets))
    mod.check_status()
    col3 = sum(t.shape[1] for t in tables[:3])
    assert torch.equal(out[:, :col3], good[:, :col3])
    # decreasing offsets are clamped and reported
    o_bad = [o.copy() for o in offsets]
    o_bad[2][10] = o_bad[2][9] - 1 if o_bad[2][9] > 0 else 0
    o_bad[2][7] = 10 ** 6
    mod(to_device(values), to_device(o_bad))
    with pytest.raises(EbError):
        mod.check_status()


def test_timing_returns_per_feature_times(cfg1):
    cfg, tables, values, offsets, mod = cfg1
    mod.set_schedules(all_schedules("flat", 4, len(tables)))
    out, times = mod(to_device(values), to_device(offsets), timing=True)
    check_against_oracle(out, tables, values, offsets, "f32")
    assert times.shape == (len(tables),) and times.dtype == torch.float64
    assert torch.all(times > 0)
    out, times = mod(to_device(values), to_device(offsets), timing=True, timing_schedules=3)
    assert times.shape == (3,)


def test_text_front_end_matches_reference_module_contract():
    """FeatProcessEmbed.forward(raw_data): strings in, [batch, sum(dim)] out (reference: rec_modules.py:127-140)."""
    from recflex_b200.rec_modules import FeatProcessEmbed

    rng = np.random.default_rng(11)
    shapes = [(100, 16), (57, 16), (300, 32)]
    tables = [(rng.standard_normal(s) * 0.1).astype(np.float32) for s in shapes]
    batch = 40
    raw, values, offsets = [], [], []
    for rows, _ in shapes:
        lines = []
        for _b in range(batch):
            n = int(rng.integers(0, 6))
            lines.append(",".join(str(int(x)) for x in rng.integers(0, rows, n)))
        raw.append(lines)
        v, o = oracle.parse_bags(lines)
        values.append(v)
        offsets.append(o)
    model = FeatProcessEmbed(None, 0, embed_tables=device_tables(tables))
    out = model(raw)
    check_against_oracle(out, tables, values, offsets, "f32")
    (out2, ms) = model(raw, timing_kernel=True)
    assert torch.equal(out, out2) and ms > 0


def test_synthetic_table_fill_is_bit_reproducible_on_cpu():
    cfg = synth.make_config(3, row_scale=1e-4, batch=8)
    dev = synth.make_tables_device(cfg, "cuda:0")
    torch.cuda.synchronize()
    for fs, t in list(zip(cfg.features, dev))[:12]:
        host = synth.synth_table(fs.seed, fs.rows, fs.dim, fs.dtype)
        assert np.array_equal(t.cpu().numpy().view(np.uint16), host.view(np.uint16))
    cfg = synth.make_config(1, row_scale=0.01)
    for fs, t in zip(cfg.features, synth.make_tables_device(cfg, "cuda:0")):
        assert np.array_equal(t.cpu().numpy(), synth.synth_table(fs.seed, fs.rows, fs.dim, fs.dtype))


def test_cuda_graph_capture_and_replay(cfg1):
    """The packed forward is two launches with no host round-trip: it can be captured once and replayed on new
    batches written into the same device buffers (the binding is recomputed on the device at every replay)."""
    cfg, tables, values, offsets, mod = cfg1
    mod.set_schedules(all_schedules("stream", 4, len(tables)), occupancy=4)
    batches = [synth.gen_batch(cfg, seed) for seed in (3, 4, 5)]
    packed = [synth.pack_batch(v, o) for v, o in batches]
    cap = max(len(pv) for pv, _ in packed)
    dv = torch.zeros(cap, dtype=torch.int32, device="cuda:0")
    do = torch.zeros(packed[0][1].shape, dtype=torch.int32, device="cuda:0")
    out = torch.empty((cfg.batch, mod.output_units), dtype=torch.float32, device="cuda:0")
    dv[: len(packed[0][0])] = torch.from_numpy(packed[0][0]).cuda()
    do.copy_(torch.from_numpy(packed[0][1]))
    mod.forward_packed(dv, do, out=out)  # warm-up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        mod.forward_packed(dv, do, out=out)
    for (v, o), (pv, po) in zip(batches, packed):
        dv[: len(pv)] = torch.from_numpy(pv).cuda()
        do.copy_(torch.from_numpy(po))
        graph.replay()
        torch.cuda.synchronize()
        check_against_oracle(out, tables, v, o, "f32")


@pytest.mark.parametrize("kind", KINDS)
def test_int64_every_kind(kind):
    cfg, tables, values, offsets = small_model(3, 2e-4, 300)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    mod.set_schedules(all_schedules(kind, 8, len(tables)))  # 64-bit indices always run at unroll 4
    out = mod(to_device(values, dtype=np.int64), to_device(offsets, dtype=np.int64))
    mod.check_status()
    check_against_oracle(out, tables, values, offsets, "f16")


def test_random_models_every_kind():
    """Fuzz: random dims (also not multiples of 4), dtypes, table sizes, length patterns, batch sizes, mixed kinds."""
    rng = np.random.default_rng(2024)
    for trial in range(24):
        F = int(rng.integers(1, 9))
        batch = int(rng.choice([1, 2, 17, 32, 33, 64, 100, 257]))
        tables, values, offsets, scheds = [], [], [], []
        for f in range(F):
            dim = int(rng.choice([1, 2, 3, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 320, 512]))
            rows = int(rng.integers(1, 2000))
            dt = np.float16 if rng.random() < 0.5 else np.float32
            tables.append((rng.standard_normal((rows, dim)) * 0.1).astype(dt))
            mode = int(rng.integers(0, 5))
            if mode == 0:
                lens = np.ones(batch, dtype=np.int64)
            elif mode == 1:
                lens = rng.integers(0, 3, batch)
            elif mode == 2:
                lens = rng.integers(0, 40, batch)
            elif mode == 3:
                lens = (rng.pareto(0.7, batch)).astype(np.int64).clip(0, 600)
            else:
                lens = np.zeros(batch, dtype=np.int64)
            o = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
            offsets.append(o)
            values.append(rng.integers(0, rows, o[-1]).astype(np.int32))
            scheds.append(Schedule(str(rng.choice(KINDS)), int(rng.choice([1, 2, 4, 8]))))
        mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
        mod.set_schedules(scheds, occupancy=int(rng.integers(1, 9)))
        out = mod(to_device(values), to_device(offsets))
        mod.check_status()
        expect = oracle.pool(tables, values, offsets, acc64=True)
        np.testing.assert_allclose(out.cpu().numpy(), expect, rtol=2e-3, atol=2e-5,
                                   err_msg=f"trial {trial}: {[(t.shape, t.dtype) for t in tables]} {scheds}")


@pytest.mark.parametrize("F", [1, 31, 32, 33, 1100])
def test_feature_counts_around_the_ticket_search_rounds(F):
    """The ticket's feature is found by probing 32 positions of the tile prefix sum per round: one round up to 32
    features, two up to 1024, three beyond.  Features on the warp-per-bag schedule own no tiles of the fused kernel, so
    the prefix sum holds runs of equal values that the search has to step over."""
    rng = np.random.default_rng(77 + F)
    batch = 70
    tables, values, offsets, scheds = [], [], [], []
    for f in range(F):
        dim = int(rng.choice([4, 8, 16, 32]))
        rows = int(rng.integers(4, 200))
        tables.append((rng.standard_normal((rows, dim)) * 0.1).astype(np.float32))
        lens = rng.integers(0, 6, batch)
        o = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        offsets.append(o)
        values.append(rng.integers(0, rows, o[-1]).astype(np.int32))
        scheds.append(Schedule("warp" if f % 5 == 3 else str(rng.choice(["pipe", "stream", "group"])), 4))
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    mod.set_schedules(scheds, occupancy=4)
    out = mod(to_device(values), to_device(offsets))
    mod.check_status()
    expect = oracle.pool(tables, values, offsets, acc64=True)
    np.testing.assert_allclose(out.cpu().numpy(), expect, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [np.int32, np.int64])
def test_offsets_from_lengths_on_device(cfg1, dtype):
    cfg, tables, values, offsets, mod = cfg1
    for batch in (1, 255, 1024, 5000):
        rng = np.random.default_rng(batch)
        lens = rng.integers(0, 9, (len(tables), batch)).astype(dtype)
        got = mod.offsets_from_lengths(torch.from_numpy(lens).cuda()).cpu().numpy()
        expect = np.concatenate([np.zeros((len(tables), 1), dtype=dtype), np.cumsum(lens, axis=1, dtype=dtype)], axis=1)
        assert got.dtype == dtype and np.array_equal(got, expect)
    # lengths -> offsets -> packed forward equals the list forward
    mod.set_schedules(all_schedules("stream", 4, len(tables)), occupancy=4)
    pv, po = synth.pack_batch(values, offsets)
    lens = torch.from_numpy(np.diff(po, axis=1).astype(dtype)).cuda()
    out = mod.forward_packed(torch.from_numpy(pv.astype(dtype)).cuda(), mod.offsets_from_lengths(lens))
    check_against_oracle(out, tables, values, offsets, "f32")


@pytest.mark.parametrize("kind", ["stream", "pipe", "warp", "flat"])
@pytest.mark.parametrize("idt", [np.int32, np.int64])
def test_long_bags(kind, idt):
    """Bags of more than a thousand entries for every dim class (1 to 32 row slots per warp, and rows wider than a
    warp), both table dtypes, 32- and 64-bit indices at every unroll (with 64-bit indices the pipelined schedule runs
    its 12-cell variant whatever unroll was requested: its ring must be sized for that), an empty bag in between,
    a bad index."""
    rng = np.random.default_rng(77)
    dims = [4, 8, 16, 32, 64, 128, 256, 8, 16, 32, 64, 128, 256, 512]
    dts = [np.float32] * 7 + [np.float16] * 7
    batch = 37
    tables, values, offsets = [], [], []
    for d, dt in zip(dims, dts):
        rows = 300
        tables.append((rng.standard_normal((rows, d)) * 0.05).astype(dt))
        lens = rng.integers(1100, 1400, batch)
        lens[5] = 0
        o = np.concatenate([[0], np.cumsum(lens)]).astype(idt)
        offsets.append(o)
        values.append(rng.integers(0, rows, o[-1]).astype(idt))
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    for unroll, occ in ((4, 8), (2, 4), (8, 3)):
        mod.set_schedules(all_schedules(kind, unroll, len(dims)), occupancy=occ)
        out = mod(to_device(values), to_device(offsets))
        mod.check_status()
        expect = oracle.pool(tables, values, offsets, acc64=True)
        np.testing.assert_allclose(out.cpu().numpy(), expect, rtol=2e-3, atol=2e-5)
    bad = [v.copy() for v in values]
    bad[2][1500] = 10 ** 6
    out = mod(to_device(bad), to_device(offsets))
    from recflex_b200._lib import EbError

    with pytest.raises(EbError):
        mod.check_status()
    good = [v.copy() for v in values]
    expect = oracle.pool(tables, bad, offsets, acc64=True, strict=False)  # the oracle skips the bad entry too
    np.testing.assert_allclose(out.cpu().numpy(), expect, rtol=2e-3, atol=2e-5)


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("interleave", [True, False])
def test_peer_mode_on_one_device(kind, interleave):
    """eb_forward_peers with every rank's output matrix on this GPU: sample b must land in matrix b // rows at row
    b % rows, whether a feature's tiles are dealt round-robin over the destinations or walked in batch order."""
    world, rows = 4, 512
    cfg, tables, values, offsets = small_model(2, 0.01, world * rows)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    mod.set_schedules(all_schedules(kind, 4, len(tables)))
    mod.set_peer_interleave(interleave)
    units = mod.output_units
    outs = [torch.full((rows, units), float("nan"), device="cuda:0") for _ in range(world)]
    mod.forward_peers(to_device(values), to_device(offsets), [o.data_ptr() for o in outs], units)
    torch.cuda.synchronize()
    mod.check_status()
    check_against_oracle(torch.cat(outs), tables, values, offsets, "f32")


def test_peer_mode_with_tiles_wider_than_a_rank():
    """Tiles that straddle two ranks' rows (bags_per_tile does not divide batch / world) keep batch order."""
    world, rows = 4, 96
    cfg, tables, values, offsets = small_model(1, 1.0, world * rows)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    mod.set_schedules(all_schedules("stream", 4, len(tables), bags_per_tile=64))
    units = mod.output_units
    outs = [torch.full((rows, units), float("nan"), device="cuda:0") for _ in range(world)]
    mod.forward_peers(to_device(values), to_device(offsets), [o.data_ptr() for o in outs], units)
    torch.cuda.synchronize()
    check_against_oracle(torch.cat(outs), tables, values, offsets, "f32")


@pytest.mark.parametrize("fused_ctas", [1, 2, 4])
def test_warp_kernel_beside_the_fused_kernel(fused_ctas):
    """Overlap mode: features on the warp-per-bag schedule are pooled on the handle's own stream while the fused
    kernel pools the rest on a reduced grid; results and stream order as seen by the caller do not change."""
    cfg, tables, values, offsets = small_model(5, 0.01, 2048)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    scheds = [Schedule("warp", 4) if f % 3 == 0 else Schedule("pipe" if f % 3 == 1 else "stream", 4)
              for f in range(len(tables))]
    mod.set_schedules(scheds, occupancy=4)
    mod.set_kernel_overlap(fused_ctas)
    dv, do = to_device(values), to_device(offsets)
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        out = None
        for _ in range(3):  # back-to-back calls reuse the workspace: each must wait for both kernels of the last
            out = mod(dv, do)
        doubled = out * 2.0  # ordered after both kernels through the caller's stream alone
    st.synchronize()
    mod.check_status()
    check_against_oracle(out, tables, values, offsets, "f32")
    assert torch.equal(doubled, out * 2.0)
    mod.set_kernel_overlap(0)  # back to one kernel after the other (tile sizes, hence summation order, may differ)
    again = mod(dv, do)
    torch.cuda.synchronize()
    check_against_oracle(again, tables, values, offsets, "f32")
