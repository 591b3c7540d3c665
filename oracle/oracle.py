"""Python face of the CPU oracle — TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference
arms may import this module; nothing under recflex_b200/ does.  `pool` calls
the C restatement in eb_oracle.c (see that file's header for the reference
lines it follows and how parity is pinned); `pool_numpy` is an independent
restatement of the same definition (examples/test.py:68-86 of the reference)
in numpy, and `pool_torch` is `torch.nn.functional.embedding_bag(mode='sum')`
on the CPU, the host baseline the benchmark definition names.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import List, Sequence, Tuple

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile eb_oracle.c with gcc (through oracle/Makefile) if the library is missing or stale."""
    src = os.path.join(HERE, "eb_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return LIB


def _load() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        lib = C.CDLL(LIB)
        lib.oracle_pool_feature.restype = C.c_int
        lib.oracle_pool_feature.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p,
                                            C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int]
        lib.oracle_parse_bags.restype = C.c_int64
        lib.oracle_parse_bags.argtypes = [C.c_char_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p]
        lib.oracle_synth_rows.restype = None
        lib.oracle_synth_rows.argtypes = [C.c_uint64, C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_void_p]
        _lib = lib
    return _lib


def _ptr(a: np.ndarray) -> C.c_void_p:
    return a.ctypes.data_as(C.c_void_p)


def pool(tables: Sequence[np.ndarray], values: Sequence[np.ndarray], offsets: Sequence[np.ndarray],
         acc64: bool = False, strict: bool = True) -> np.ndarray:
    """Expected output [batch, sum(dim)] fp32.  tables[f]: [rows, dim] float32 or float16;
    values[f]: indices; offsets[f]: batch + 1 boundaries."""
    lib = _load()
    batch = len(offsets[0]) - 1
    units = sum(t.shape[1] for t in tables)
    out = np.zeros((batch, units), dtype=np.float32)
    col = 0
    for t, v, o in zip(tables, values, offsets):
        t = np.ascontiguousarray(t)
        v64 = np.ascontiguousarray(v, dtype=np.int64)
        o64 = np.ascontiguousarray(o, dtype=np.int64)
        assert len(o64) == batch + 1
        f16 = t.dtype == np.float16
        assert f16 or t.dtype == np.float32
        rc = lib.oracle_pool_feature(_ptr(t), int(f16), t.shape[0], t.shape[1], _ptr(v64), _ptr(o64), batch,
                                     _ptr(out), units, col, int(acc64))
        if rc != 0 and strict:
            raise ValueError("index or offset out of range")
        col += t.shape[1]
    return out


def pool_numpy(tables: Sequence[np.ndarray], values: Sequence[np.ndarray], offsets: Sequence[np.ndarray]) -> np.ndarray:
    """Independent numpy restatement: per bag, gather the rows and sum them (float64 accumulate)."""
    batch = len(offsets[0]) - 1
    cols = []
    for t, v, o in zip(tables, values, offsets):
        res = np.zeros((batch, t.shape[1]), dtype=np.float64)
        gathered = t[np.asarray(v, dtype=np.int64)].astype(np.float64)
        o = np.asarray(o, dtype=np.int64)
        # loop the bags: differences of a running sum would lose bits
        for b in range(batch):
            if o[b + 1] > o[b]:
                res[b] = gathered[o[b]:o[b + 1]].sum(axis=0)
        cols.append(res)
    return np.concatenate(cols, axis=1).astype(np.float32)


def pool_torch(tables: Sequence, values: Sequence, offsets: Sequence, threads: int = 0):
    """torch.nn.functional.embedding_bag(mode='sum') per feature on the CPU, concatenated.
    fp16 tables are up-cast to fp32 first (fp32 accumulation)."""
    import torch
    import torch.nn.functional as F

    if threads:
        torch.set_num_threads(threads)
    outs = []
    for t, v, o in zip(tables, values, offsets):
        t = torch.as_tensor(t)
        if t.dtype != torch.float32:
            t = t.float()
        v = torch.as_tensor(v).long()
        o = torch.as_tensor(o).long()
        outs.append(F.embedding_bag(v, t, o, mode="sum", include_last_offset=True))
    return torch.cat(outs, dim=1)


def parse_bags(lines: Sequence[str]) -> Tuple[np.ndarray, np.ndarray]:
    lib = _load()
    text = "\n".join(lines).encode()
    cap = len(text) + 1
    values = np.empty(cap, dtype=np.int32)
    offsets = np.empty(len(lines) + 1, dtype=np.int32)
    n = lib.oracle_parse_bags(text, len(text), len(lines), _ptr(values), cap, _ptr(offsets))
    assert n >= 0
    return values[:n].copy(), offsets


def synth_rows(seed: int, row_ids: np.ndarray, dim: int, std: float = 0.01) -> np.ndarray:
    lib = _load()
    ids = np.ascontiguousarray(row_ids, dtype=np.int64)
    out = np.empty((len(ids), dim), dtype=np.float32)
    lib.oracle_synth_rows(seed, _ptr(ids), len(ids), dim, std, _ptr(out))
    return out
