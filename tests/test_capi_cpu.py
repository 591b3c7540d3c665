"""CPU: the C-ABI library loads, exports every symbol the header declares, and fails loudly without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    with open(os.path.join(ROOT, "include", "recflex_b200.h")) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(eb_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    from recflex_b200 import _lib

    names = header_functions()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.PROTOTYPES) == names, "ctypes prototypes and header disagree"
    assert b"sm_100a" in lib.eb_version()


def test_header_constants_match_binding():
    from recflex_b200 import _lib

    with open(os.path.join(ROOT, "include", "recflex_b200.h")) as f:
        text = f.read()
    defs = dict(re.findall(r"#define\s+(EB_[A-Z0-9_]+)\s+\(?(-?\d+)\)?", text))
    for name, value in defs.items():
        assert getattr(_lib, name) == int(value), name


def test_parse_bags_errors(lib):
    from recflex_b200 import _lib

    vals = np.zeros(2, dtype=np.int32)
    offs = np.zeros(3, dtype=np.int32)
    nnz = C.c_int64()
    text = b"1,2,3\n4"
    rc = lib.eb_parse_bags(text, len(text), 2, vals.ctypes.data_as(C.c_void_p), 2, offs.ctypes.data_as(C.c_void_p),
                           C.byref(nnz))
    assert rc == _lib.EB_ERR_WORKSPACE_TOO_SMALL
    assert b"values_out" in lib.eb_last_error()
    rc = lib.eb_parse_bags(text, len(text), -1, None, 0, offs.ctypes.data_as(C.c_void_p), C.byref(nnz))
    assert rc == _lib.EB_ERR_INVALID_ARG
    with pytest.raises(_lib.EbError):
        _lib.check(rc)


def test_no_fallback_without_gpu(lib):
    """Without a CUDA device the product path must fail, not fall back."""
    import torch

    from recflex_b200 import _lib
    from recflex_b200.rec_modules import FeatEmbed

    with pytest.raises(ValueError):
        FeatEmbed("cpu", table_shapes=[(4, 4)])
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rows = (C.c_int64 * 1)(4)
    dims = (C.c_int32 * 1)(4)
    dts = (C.c_int32 * 1)(0)
    ptrs = (C.c_void_p * 1)(16)
    rc = lib.eb_create(C.byref(h), 0, 1, rows, dims, dts, ptrs)
    assert rc == _lib.EB_ERR_CUDA and not h.value


def test_argument_validation_needs_no_gpu(lib):
    from recflex_b200 import _lib

    h = C.c_void_p()
    assert lib.eb_create(C.byref(h), 0, 0, None, None, None, None) == _lib.EB_ERR_INVALID_ARG
    assert lib.eb_create(None, 0, 1, None, None, None, None) == _lib.EB_ERR_INVALID_ARG
    assert lib.eb_workspace_bytes(None, None) == _lib.EB_ERR_INVALID_ARG
    assert lib.eb_forward_packed_noalloc(0, _lib.EB_NOALLOC_MAX_FEATURES + 1, None, None, None, None, 1, None, None, 0,
                                         None, 0, None) == _lib.EB_ERR_TOO_LARGE
