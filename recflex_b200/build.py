"""Build librecflex_b200.so in-tree with nvcc for sm_100a.

Run `python -m recflex_b200.build` (or call `build()`).  The fused kernel is
compiled once per CTAs-per-SM occupancy; those translation units are
independent and build in parallel.  Objects land in `recflex_b200/build/`, the
library beside the package as `recflex_b200/librecflex_b200.so`.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
BUILD_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "librecflex_b200.so")
INCLUDE_DIR = os.path.join(os.path.dirname(PKG_DIR), "include")

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return nvcc


def _sources_digest() -> str:
    h = hashlib.sha256()
    names = sorted(os.listdir(CSRC)) + ["../../include/recflex_b200.h"]
    for name in names:
        path = os.path.normpath(os.path.join(CSRC, name))
        if os.path.isfile(path):
            h.update(name.encode())
            with open(path, "rb") as f:
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _units():
    """(object name, source, extra flags)"""
    units = [
        ("eb_capi.o", "eb_capi.cu", []),
        ("eb_launch.o", "eb_launch.cu", []),
        ("eb_noalloc.o", "eb_noalloc.cu", []),
        ("eb_warp.o", "eb_warp_inst.cu", []),
        ("eb_longbag.o", "eb_longbag_inst.cu", []),
    ]
    for occ in range(1, 9):
        units.append((f"eb_fused_occ{occ}.o", "eb_fused_inst.cu", [f"-DEB_OCC={occ}"]))
    return [u for u in units if os.path.exists(os.path.join(CSRC, u[1]))]


def _compile(unit, verbose: bool) -> str:
    obj, src, extra = unit
    out = os.path.join(BUILD_DIR, obj)
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-I", INCLUDE_DIR, "-c", os.path.join(CSRC, src), "-o", out]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src} {extra}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return out


def build(force: bool = False, verbose: bool = False, jobs: int | None = None) -> str:
    """Compile (if sources changed) and return the path of the shared library."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    stamp = os.path.join(BUILD_DIR, "sources.sha256")
    digest = _sources_digest()
    if not force and os.path.exists(LIB_PATH) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return LIB_PATH
    units = _units()
    jobs = jobs or min(len(units), os.cpu_count() or 1)
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs) as pool:
        objs = list(pool.map(lambda u: _compile(u, verbose), units))
    cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
