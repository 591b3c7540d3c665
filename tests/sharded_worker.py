"""Worker of the sharded-path tests: one process per rank (gloo on CPU with test hooks, or nccl on GPUs).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 --master-port P \
        tests/sharded_worker.py --backend gloo|nccl [--chunks C] [--exchange nccl|peer|copy] [--model small|cfg4]

Every rank builds the same model and batch from a seed, shards the tables with the planner, runs the sharded
forward and compares its rows with the oracle's result for the whole batch.  `--model small` is a 9-feature model
with mixed dims and dtypes; `--model cfg4` is the sharded benchmark configuration scaled down (400 features, the
benchmark's own planner call, ranks with about 400 / world tables each).  With gloo the pooling and placement
hooks are the CPU oracle / torch (test infrastructure); with nccl the product path runs.
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np
import torch
import torch.distributed as dist

from oracle import oracle
from recflex_b200.sharding import ShardedFeatEmbed, local_sample_ids, plan_shards, shard_summary


def small_model(backend, B):
    rng = np.random.default_rng(123)
    dims = [16, 4, 64, 8, 32, 128, 16, 256, 8]
    rows = [50, 1000, 70, 33, 400, 90, 64, 20, 5000]
    dtypes = [np.float32, np.float16]
    tables = [(rng.standard_normal((r, d)) * 0.1).astype(dtypes[i % 2] if backend == "nccl" else np.float32)
              for i, (r, d) in enumerate(zip(rows, dims))]
    values, offsets = [], []
    for i, r in enumerate(rows):
        lens = rng.integers(0, 6, B) if i % 3 else np.ones(B, dtype=np.int64)
        o = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        offsets.append(o)
        values.append(rng.integers(0, r, o[-1]).astype(np.int32))
    return dims, tables, values, offsets


def cfg4_model(world, B):
    """The sharded benchmark configuration with tables scaled by 1e-4, sharded by the benchmark's own planner call."""
    import bench
    from recflex_b200 import synth

    cfg = synth.make_config(4, row_scale=1e-4, batch=B)
    tables = synth.make_tables_numpy(cfg)
    values, offsets = synth.gen_batch(cfg, seed=5)
    owner, summ = bench.plan_cfg_shards(cfg, world, cap=1 << 40)
    return [fs.dim for fs in cfg.features], tables, values, offsets, owner, summ


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="gloo")
    ap.add_argument("--chunks", type=int, default=3)
    ap.add_argument("--batch", type=int, default=48)
    ap.add_argument("--exchange", default="nccl")
    ap.add_argument("--model", default="small")
    ap.add_argument("--columns", default="owner")
    ap.add_argument("--out-dtype", default="f32")
    ap.add_argument("--direct-hops", type=int, default=0)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if args.backend == "nccl":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")

    B = args.batch
    if args.model == "cfg4":
        dims, tables, values, offsets, owner, summ = cfg4_model(world, B)
        assert len(dims) == 400 and min(np.bincount(owner, minlength=world)) >= 400 // world // 2
    else:
        dims, tables, values, offsets = small_model(args.backend, B)
        table_bytes = [t.nbytes for t in tables]
        traffic = [float(o[-1]) * t.shape[1] * t.itemsize for o, t in zip(offsets, tables)]
        owner = plan_shards(table_bytes, traffic, world)
        summ = shard_summary(owner, table_bytes, traffic, world)
    assert sorted(set(owner)) == list(range(world)), owner
    local = [f for f, r in enumerate(owner) if r == rank]
    out_dtype = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[args.out_dtype]

    if args.backend == "nccl":
        mod = ShardedFeatEmbed(rank, world, owner, dims, local_tables=[torch.from_numpy(tables[f]).to(dev) for f in local],
                               device=dev, chunks=args.chunks, exchange=args.exchange, out_dtype=out_dtype,
                               columns=args.columns, direct_hops=args.direct_hops)
        lv = [torch.from_numpy(values[f]).to(dev) for f in local]
        lo = [torch.from_numpy(offsets[f]).to(dev) for f in local]
    else:
        def pool_fn(vals, offs, out):
            res = oracle.pool([tables[f] for f in local], [v.numpy() for v in vals], [o.numpy() for o in offs])
            out[:, : res.shape[1]] = torch.from_numpy(res)

        def place_fn(recv, out_k, nrows):
            for so, sl, dc, w in mod.segments(nrows):
                block = recv[so: so + (nrows - 1) * sl + w]
                for rr in range(nrows):
                    out_k[rr, dc: dc + w] = block[rr * sl: rr * sl + w]

        mod = ShardedFeatEmbed(rank, world, owner, dims, chunks=args.chunks, pool_fn=pool_fn, place_fn=place_fn)
        lv = [torch.from_numpy(values[f]) for f in local]
        lo = [torch.from_numpy(offsets[f]) for f in local]
    mod.set_batch_for_empty_rank(B)
    cat = (lambda t: torch.cat(t, dim=1)) if args.columns == "blocks" else (lambda t: t)
    out = cat(mod(lv, lo))
    if args.backend == "nccl":
        torch.cuda.synchronize()
    chunks_eff = args.chunks if args.exchange == "nccl" else 1  # the other exchanges split the batch contiguously
    canon = oracle.pool(tables, values, offsets, acc64=True)[local_sample_ids(B, world, chunks_eff, rank)]
    expect = np.empty_like(canon)
    col = 0
    for f, d in enumerate(dims):  # feature f's columns sit where the module says
        expect[:, mod.column_of[f]: mod.column_of[f] + d] = canon[:, col: col + d]
        col += d
    if args.exchange == "copy" and args.columns != "canonical" and world > 1 and args.model == "small":
        assert mod.column_of != mod.col_of, "owner-major columns should differ from feature order here"
    rtol, atol = (2e-3, 1e-5) if args.backend == "nccl" else (1e-5, 1e-5)
    if out_dtype != torch.float32:
        rtol, atol = 1.0 / 64, 1e-3  # one rounding to 8 (bf16) or 11 (f16) significant bits, twice for cut bags
    np.testing.assert_allclose(out.float().cpu().numpy(), expect, rtol=rtol, atol=atol)
    # a second call reuses the buffers
    out2 = cat(mod(lv, lo))
    if args.backend == "nccl":
        torch.cuda.synchronize()
    assert torch.equal(out, out2)
    out3 = cat(mod(lv, lo))  # peer and copy exchanges: a third call is back on the first of the two buffers
    assert torch.equal(out3, out2)
    dist.barrier()
    if args.backend == "nccl":
        mod.close()
    if rank == 0:
        print("sharded ok", args.backend, "world", world, "imbalance %.3f" % summ["traffic_imbalance"], flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
