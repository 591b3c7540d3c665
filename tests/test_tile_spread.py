"""The peer exchange's tile-to-destination mapping (host/device function `ebk::spread_tile`), checked on the host."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_spread_tile_is_a_bijection_that_interleaves_ranks(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    exe = tmp_path / "spread_check"
    build = subprocess.run([nvcc, "-O1", "-std=c++17", "-I", os.path.join(ROOT, "recflex_b200", "csrc"), "-o", str(exe),
                            os.path.join(ROOT, "tests", "spread_check.cu")], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout
    assert run.stdout.startswith("ok ")
