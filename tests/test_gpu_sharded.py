"""GPU (2 or more devices): the product sharded forward over NCCL / NVLink peer memory against the oracle."""
import pytest
import torch

from tests.test_sharding import run_workers

pytestmark = pytest.mark.gpu


def _world():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    return 4 if n >= 4 else 2


def _run(world, extra):
    res = run_workers(world, "nccl", extra)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert f"sharded ok nccl world {world}" in res.stdout


@pytest.mark.parametrize("chunks", [1, 4])
def test_sharded_forward_nccl(chunks):
    world = _world()
    _run(world, ["--chunks", str(chunks), "--batch", str(world * chunks * 6)])


def test_sharded_forward_fused_peer_exchange():
    world = _world()
    _run(world, ["--exchange", "peer", "--batch", str(world * 1024)])


@pytest.mark.parametrize("columns", ["owner", "canonical", "blocks"])
def test_sharded_forward_copy_engine_exchange(columns):
    world = _world()
    _run(world, ["--exchange", "copy", "--chunks", "4", "--batch", str(world * 1024), "--columns", columns])


@pytest.mark.parametrize("exchange,chunks", [("peer", 1), ("copy", 8), ("push", 8), ("nccl", 4)])
def test_sharded_cfg4_shaped_plan(exchange, chunks):
    """The sharded benchmark configuration scaled down: 400 features, the benchmark's planner call, every exchange."""
    world = _world()
    _run(world, ["--model", "cfg4", "--exchange", exchange, "--chunks", str(chunks), "--batch", str(world * 1024)])


def test_sharded_bf16_rows_through_both_fused_exchanges():
    world = _world()
    _run(world, ["--exchange", "peer", "--batch", str(world * 512), "--out-dtype", "bf16"])
    _run(world, ["--exchange", "copy", "--chunks", "2", "--batch", str(world * 512), "--out-dtype", "bf16"])


def test_sharded_hybrid_exchange_stores_to_the_nearest_rank_and_copies_to_the_rest():
    world = _world()
    _run(world, ["--exchange", "copy", "--chunks", "4", "--batch", str(world * 1024), "--columns", "blocks",
                 "--direct-hops", str(max(1, world // 2))])
