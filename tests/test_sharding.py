"""CPU: the shard planner, and the sharded forward's exchange/placement logic on two gloo ranks."""
import os
import socket
import subprocess
import sys

import pytest

from recflex_b200.sharding import ShardedFeatEmbed, local_sample_ids, plan_shards, shard_summary

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_workers(world, backend, extra=()):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "sharded_worker.py"), "--backend", backend, *extra]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)


def test_planner_balances_traffic_under_capacity():
    import numpy as np

    rng = np.random.default_rng(0)
    F, W = 400, 8
    table_bytes = [int(x) for x in np.exp(rng.uniform(np.log(1e6), np.log(1e10), F))]
    traffic = [float(x) for x in np.exp(rng.uniform(np.log(1e3), np.log(1e7), F))]
    cap = int(sum(table_bytes) / W * 1.3)
    owner = plan_shards(table_bytes, traffic, W, cap)
    s = shard_summary(owner, table_bytes, traffic, W)
    assert max(s["bytes_per_rank"]) <= cap
    assert s["traffic_imbalance"] < 1.05
    assert set(owner) == set(range(W))
    # deterministic
    assert owner == plan_shards(table_bytes, traffic, W, cap)


def test_planner_balances_gather_and_exchange_loads():
    """With the second load (pooled bytes each owner sends) the planner evens out both; the single-load plan of
    the sharded benchmark configuration leaves one rank sending 13 % more than the mean."""
    from recflex_b200 import synth

    W = 8
    cfg = synth.make_config(4)
    table_bytes = [fs.table_bytes for fs in cfg.features]
    traffic = synth.expected_traffic(cfg)
    sent = [cfg.batch * fs.dim * 4 * (W - 1) / W for fs in cfg.features]
    cap = int(1.15 * sum(table_bytes) / W)
    one = shard_summary(plan_shards(table_bytes, traffic, W, int(168e9)), table_bytes, traffic, W, exchange=sent)
    owner = plan_shards(table_bytes, traffic, W, cap, exchange=sent)
    two = shard_summary(owner, table_bytes, traffic, W, exchange=sent)
    assert one["exchange_imbalance"] > 1.10
    assert two["exchange_imbalance"] < 1.01 and two["traffic_imbalance"] < 1.01
    assert max(two["bytes_per_rank"]) <= cap and set(owner) == set(range(W))
    assert owner == plan_shards(table_bytes, traffic, W, cap, exchange=sent)  # deterministic
    with pytest.raises(ValueError):
        plan_shards(table_bytes, traffic, W, cap, exchange=sent[:-1])


def test_planner_capacity_errors():
    with pytest.raises(ValueError):
        plan_shards([10, 10], [1.0, 1.0], 2, capacity_bytes=5)
    with pytest.raises(ValueError):
        plan_shards([6, 6, 6], [1.0, 1.0, 1.0], 2, capacity_bytes=10)
    assert sorted(plan_shards([6, 6], [1.0, 1.0], 2, capacity_bytes=10)) == [0, 1]


def test_layout_helpers():
    m = ShardedFeatEmbed(0, 2, [0, 1, 0, 1], [4, 8, 16, 4], pool_fn=lambda *a: None, place_fn=lambda *a: None)
    assert m.units == 32 and m.units_of == [20, 12] and m.local_features == [0, 2]
    segs = m.segments(3)
    # rank 0's block [3, 20] first (features 0, 2), then rank 1's block [3, 12] (features 1, 3)
    assert segs == [(0, 20, 0, 4), (4, 20, 12, 16), (60, 12, 4, 8), (68, 12, 28, 4)]
    assert local_sample_ids(24, 2, 3, 1) == [4, 5, 6, 7, 12, 13, 14, 15, 20, 21, 22, 23]
    with pytest.raises(ValueError):
        ShardedFeatEmbed(0, 2, [0, 1], [4, 4])  # product path without CUDA tables: no fallback


@pytest.mark.parametrize("chunks", [1, 3])
def test_sharded_forward_two_gloo_ranks(chunks):
    res = run_workers(2, "gloo", ["--chunks", str(chunks)])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "sharded ok gloo world 2" in res.stdout


def test_sharded_cfg4_shaped_plan_two_gloo_ranks():
    """Host logic on the sharded benchmark configuration scaled down (400 features, the benchmark's planner call)."""
    res = run_workers(2, "gloo", ["--model", "cfg4", "--chunks", "2", "--batch", "24"])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "sharded ok gloo world 2" in res.stdout
