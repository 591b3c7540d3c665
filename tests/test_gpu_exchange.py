"""GPU, one device: the two fused exchanges of the sharded path with every rank's buffers on this GPU.

The ranks of a table-wise sharding are played one after the other by modules that each own one rank's tables;
their pooled rows go to `world` result matrices that all live on this device.  That exercises exactly what a
rank runs on a multi-GPU box (the planner's assignment, the column layouts with gaps, the chunked tile order with
its device flags, the copy stream's waits and 2-D copies) except the NVLink hop itself, which
tests/test_gpu_sharded.py covers on boxes with two or more GPUs.
"""
import numpy as np
import pytest
import torch

import bench
from oracle import oracle
from recflex_b200 import synth
from recflex_b200.rec_modules import FeatEmbed, Schedule
from tests.helpers import TOL

pytestmark = pytest.mark.gpu


def _cfg4_scaled(world, rows_per_rank):
    cfg = synth.make_config(4, row_scale=1e-4, batch=world * rows_per_rank)
    tables = synth.make_tables_numpy(cfg)
    values, offsets = synth.gen_batch(cfg, seed=5)
    owner, _ = bench.plan_cfg_shards(cfg, world, cap=1 << 40)
    return cfg, tables, values, offsets, owner


def _rank_module(cfg, tables, owner, rank, kind):
    local = [f for f, r in enumerate(owner) if r == rank]
    mod = FeatEmbed("cuda:0", embed_tables=[torch.from_numpy(tables[f]).cuda() for f in local])
    mod.set_schedules([Schedule(kind, 4) for _ in local], occupancy=4)
    return local, mod


@pytest.mark.parametrize("kind", ["stream", "pipe", "warp"])
@pytest.mark.parametrize("chunks", [1, 8])
@pytest.mark.parametrize("engine,direct_hops", [("copy", 0), ("push", 0), ("copy", 2), ("copy", 3)])
def test_copy_engine_exchange_on_one_device(kind, chunks, engine, direct_hops):
    world, rows = 4, 256
    cfg, tables, values, offsets, owner = _cfg4_scaled(world, rows)
    B, units = cfg.batch, cfg.output_units
    results = [torch.full((rows, units), float("nan"), device="cuda:0") for _ in range(world)]
    ptrs = [t.data_ptr() for t in results]
    copy_streams = [torch.cuda.Stream() for _ in range(2)]
    column_of, block = [0] * len(cfg.features), 0
    for rank in range(world):
        local, mod = _rank_module(cfg, tables, owner, rank, kind)
        mod.set_exchange_engine(engine)  # who ships the pieces: the copy engines, or a small kernel
        mod.set_exchange_direct(direct_hops)  # rows for the nearest ranks stored by the pooling kernel itself
        send = torch.full((B, mod.output_units), float("nan"), device="cuda:0")
        dv = [torch.from_numpy(values[f]).cuda() for f in local]
        do = [torch.from_numpy(offsets[f]).cuda() for f in local]
        for _ in range(2):  # the second call meets the flags the first one left raised
            mod.forward_exchange(dv, do, send, ptrs, rank, units, block, chunks, copy_streams)
            for cs in copy_streams:
                torch.cuda.current_stream().wait_stream(cs)
        torch.cuda.synchronize()
        mod.check_status()
        c = block
        for f in local:
            column_of[f] = c
            c += cfg.features[f].dim
        block = c
    got = torch.cat(results).cpu().numpy()
    canon = oracle.pool(tables, values, offsets, acc64=True)
    col = 0
    for f, fs in enumerate(cfg.features):
        np.testing.assert_allclose(got[:, column_of[f]:column_of[f] + fs.dim], canon[:, col:col + fs.dim], **TOL["f16"])
        col += fs.dim


@pytest.mark.parametrize("kind", ["stream", "pipe"])
def test_peer_store_exchange_with_a_cfg4_shaped_plan_on_one_device(kind):
    world, rows = 4, 256
    cfg, tables, values, offsets, owner = _cfg4_scaled(world, rows)
    units = cfg.output_units
    cols = np.concatenate([[0], np.cumsum([fs.dim for fs in cfg.features])])
    results = [torch.full((rows, units), float("nan"), device="cuda:0") for _ in range(world)]
    for rank in range(world):
        local, mod = _rank_module(cfg, tables, owner, rank, kind)
        mod.set_output_columns([int(cols[f]) for f in local], units)  # canonical columns: gaps between a rank's features
        mod.forward_peers([torch.from_numpy(values[f]).cuda() for f in local],
                          [torch.from_numpy(offsets[f]).cuda() for f in local], [t.data_ptr() for t in results], units)
        torch.cuda.synchronize()
        mod.check_status()
    got = torch.cat(results).cpu().numpy()
    np.testing.assert_allclose(got, oracle.pool(tables, values, offsets, acc64=True), **TOL["f16"])


def test_chunked_order_rejects_batches_it_cannot_split():
    cfg, tables, values, offsets, owner = _cfg4_scaled(2, 64)
    local, mod = _rank_module(cfg, tables, owner, 0, "stream")
    send = torch.empty((cfg.batch, mod.output_units), device="cuda:0")
    res = torch.empty((cfg.batch // 2, cfg.output_units), device="cuda:0")
    dv = [torch.from_numpy(values[f]).cuda() for f in local]
    do = [torch.from_numpy(offsets[f]).cuda() for f in local]
    from recflex_b200._lib import EbError

    with pytest.raises(EbError):  # 128 samples do not split into 2 ranks x 3 pieces
        mod.forward_exchange(dv, do, send, [res.data_ptr()] * 2, 0, cfg.output_units, 0, 3, [torch.cuda.Stream()])
