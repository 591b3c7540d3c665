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
