"""GPU (2 or more devices): the product sharded forward over NCCL against the oracle."""
import pytest
import torch

from tests.test_sharding import run_workers

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunks", [1, 4])
def test_sharded_forward_nccl(chunks):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 4 if n >= 4 else 2
    res = run_workers(world, "nccl", ["--chunks", str(chunks), "--batch", str(world * chunks * 6)])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert f"sharded ok nccl world {world}" in res.stdout


def test_sharded_forward_fused_peer_exchange():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 4 if n >= 4 else 2
    res = run_workers(world, "nccl", ["--exchange", "peer", "--batch", str(world * 1024)])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert f"sharded ok nccl world {world}" in res.stdout
