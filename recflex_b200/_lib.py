"""ctypes binding of librecflex_b200.so (the C ABI in include/recflex_b200.h).

There is no fallback: if the library is missing or fails to load, importing
the product path raises.  Build it with `python -m recflex_b200.build`.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "librecflex_b200.so")

EB_OK = 0
EB_ERR_INVALID_ARG = -1
EB_ERR_CUDA = -2
EB_ERR_WORKSPACE_TOO_SMALL = -3
EB_ERR_BAD_INPUT = -4
EB_ERR_UNSUPPORTED = -5
EB_ERR_TOO_LARGE = -6

EB_F32, EB_F16 = 0, 1
EB_I32, EB_I64 = 0, 1
EB_OUT_F32, EB_OUT_BF16, EB_OUT_F16 = 0, 1, 2
EB_EXCHANGE_COPY_ENGINES, EB_EXCHANGE_SM_PUSH = 0, 1
EB_NOALLOC_MAX_FEATURES = 1024
EB_SCHED_AUTO, EB_SCHED_GROUP, EB_SCHED_WARP, EB_SCHED_FLAT, EB_SCHED_STREAM, EB_SCHED_PIPE = 0, 1, 2, 3, 4, 5
SCHED_NAMES = {EB_SCHED_AUTO: "auto", EB_SCHED_GROUP: "group", EB_SCHED_WARP: "warp", EB_SCHED_FLAT: "flat",
               EB_SCHED_STREAM: "stream", EB_SCHED_PIPE: "pipe"}
SCHED_KINDS = {v: k for k, v in SCHED_NAMES.items()}


class EbSchedule(C.Structure):
    """Mirror of `eb_schedule`."""

    _fields_ = [
        ("kind", C.c_int32),
        ("unroll", C.c_int32),
        ("vec_bytes", C.c_int32),
        ("bags_per_tile", C.c_int32),
    ]


class EbError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"recflex_b200 error {code}: {message}")
        self.code = code


# name -> (restype, argtypes); every symbol the header declares
PROTOTYPES = {
    "eb_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int32),
                            C.POINTER(C.c_int32), C.POINTER(C.c_void_p)]),
    "eb_destroy": (C.c_int, [C.c_void_p]),
    "eb_output_units": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
    "eb_set_schedules": (C.c_int, [C.c_void_p, C.POINTER(EbSchedule), C.c_int]),
    "eb_get_schedules": (C.c_int, [C.c_void_p, C.POINTER(EbSchedule), C.POINTER(C.c_int)]),
    "eb_workspace_bytes": (C.c_int, [C.c_void_p, C.POINTER(C.c_size_t)]),
    "eb_max_concurrent_ctas": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int)]),
    "eb_forward": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int64),
                             C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p]),
    "eb_forward_packed": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int64,
                                    C.c_void_p, C.c_size_t, C.c_void_p]),
    "eb_forward_host": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_void_p,
                                  C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "eb_host_staging_bytes": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.POINTER(C.c_size_t)]),
    "eb_forward_timed": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                   C.POINTER(C.c_int64), C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_void_p,
                                   C.c_size_t, C.c_void_p, C.POINTER(C.c_double)]),
    "eb_kernel_timing": (C.c_int, [C.c_void_p, C.c_int]),
    "eb_kernel_times": (C.c_int, [C.c_void_p, C.POINTER(C.c_float), C.c_int, C.POINTER(C.c_int)]),
    "eb_check_status": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "eb_last_binding": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]),
    "eb_fill_table": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_uint64, C.c_float, C.c_int,
                                C.c_void_p]),
    "eb_set_output_columns": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_int64]),
    "eb_forward_peers": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                   C.POINTER(C.c_int64), C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_int, C.c_int64,
                                   C.c_void_p, C.c_size_t, C.c_void_p]),
    "eb_set_peer_interleave": (C.c_int, [C.c_void_p, C.c_int]),
    "eb_set_kernel_overlap": (C.c_int, [C.c_void_p, C.c_int]),
    "eb_peer_alloc": (C.c_int, [C.c_int, C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]),
    "eb_peer_open": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]),
    "eb_peer_close": (C.c_int, [C.c_int, C.c_void_p]),
    "eb_peer_free": (C.c_int, [C.c_int, C.c_void_p]),
    "eb_place_columns": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_int,
                                   C.c_void_p]),
    "eb_offsets_from_lengths": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "eb_parse_bags": (C.c_int, [C.c_char_p, C.c_size_t, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                C.POINTER(C.c_int64)]),
    "eb_forward_packed_noalloc": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int32),
                                            C.POINTER(C.c_int32), C.POINTER(C.c_void_p), C.c_int64, C.c_void_p,
                                            C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_void_p]),
    "eb_noalloc_check_status": (C.c_int, [C.c_int, C.c_void_p]),
    "eb_set_output_dtype": (C.c_int, [C.c_void_p, C.c_int]),
    "eb_set_long_bag_split": (C.c_int, [C.c_void_p, C.c_int64]),
    "eb_set_exchange_engine": (C.c_int, [C.c_void_p, C.c_int]),
    "eb_set_exchange_direct": (C.c_int, [C.c_void_p, C.c_int]),
    "eb_forward_exchange": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                      C.POINTER(C.c_int64), C.c_int, C.c_int, C.c_void_p, C.c_int64,
                                      C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int,
                                      C.c_void_p, C.c_size_t, C.c_void_p, C.POINTER(C.c_void_p), C.c_int]),
    "eb_last_error": (C.c_char_p, []),
    "eb_version": (C.c_char_p, []),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (once) and attach the prototypes.  Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build the CUDA library with `python -m recflex_b200.build` "
            "(there is no CPU or PyTorch fallback for the fused embedding-bag forward)"
        )
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code: int) -> None:
    """Raise EbError for a negative status."""
    if code != EB_OK:
        msg = load().eb_last_error()
        raise EbError(code, msg.decode() if msg else "")
