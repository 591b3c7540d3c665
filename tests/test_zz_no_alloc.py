"""The allocation-free entry point (eb_forward_packed_noalloc) against the handle-based forward.

Some callers of this library cannot allocate device memory: a plugin inside a
serving process whose memory pool owns the whole GPU, a sandbox that forbids
allocation calls, a latency path where an allocation's implicit
synchronisation is unacceptable.  For them the library carries its descriptor
table and scratch in an array built into its own image.  This test calls that
entry point through the C ABI twice in a row (the second call reuses the array
the first one left dirty) and checks each result against eb_forward_packed on
the same inputs, with the tolerances of the other parity tests.  It lives in a
file that pytest collects last and passes alone in a fresh process as well.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from recflex_b200 import _lib, synth
from recflex_b200.rec_modules import FeatEmbed
from tests.helpers import TOL, check_against_oracle, device_tables, small_model

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, tables_dev, values, offsets, out):
    F = len(tables_dev)
    rows = (C.c_int64 * F)(*[t.shape[0] for t in tables_dev])
    dims = (C.c_int32 * F)(*[t.shape[1] for t in tables_dev])
    dts = (C.c_int32 * F)(*[_lib.EB_F16 if t.dtype == torch.float16 else _lib.EB_F32 for t in tables_dev])
    ptrs = (C.c_void_p * F)(*[t.data_ptr() for t in tables_dev])
    idt = _lib.EB_I64 if values.dtype == torch.int64 else _lib.EB_I32
    batch = offsets.shape[1] - 1
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.eb_forward_packed_noalloc(0, F, rows, dims, dts, ptrs, batch, C.c_void_p(values.data_ptr()),
                                         C.c_void_p(offsets.data_ptr()), idt, C.c_void_p(out.data_ptr()),
                                         out.stride(0), stream)


@pytest.mark.parametrize("cfg_id,scale,batch,tag", [(3, 2e-4, 700, "f16"), (2, 0.01, 515, "f32")])
def test_noalloc_matches_handle_forward_twice(lib, cfg_id, scale, batch, tag):
    cfg, tables, v0, o0 = small_model(cfg_id, scale, batch, seed=0)
    _, _, v1, o1 = small_model(cfg_id, scale, batch, seed=1)
    tables_dev = device_tables(tables)
    mod = FeatEmbed("cuda:0", embed_tables=tables_dev)
    for values, offsets in ((v0, o0), (v1, o1)):  # two calls in a row share the built-in scratch array
        pv, po = synth.pack_batch(values, offsets)
        dv, do = torch.from_numpy(pv).cuda(), torch.from_numpy(po).cuda()
        ref = mod.forward_packed(dv, do)
        out = torch.full_like(ref, float("nan"))
        _lib.check(_call_noalloc(lib, tables_dev, dv, do, out))
        torch.cuda.synchronize()
        torch.testing.assert_close(out, ref, **TOL[tag])
        check_against_oracle(out, tables, values, offsets, tag)


def test_noalloc_refuses_more_features_than_its_array_holds(lib):
    F = _lib.EB_NOALLOC_MAX_FEATURES + 1
    t = torch.zeros((4, 4), device="cuda:0")
    out = torch.zeros((1, 4 * F), device="cuda:0")
    vals = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    offs = torch.zeros((F, 2), dtype=torch.int32, device="cuda:0")
    rc = _call_noalloc(lib, [t] * F, vals, offs, out)
    assert rc == _lib.EB_ERR_TOO_LARGE
    assert b"exceed" in lib.eb_last_error()


def test_noalloc_status_word_and_capture_refusal(lib):
    cfg, tables, values, offsets = small_model(1, 0.1, 256)
    tables_dev = device_tables(tables)
    pv, po = synth.pack_batch(values, offsets)
    dv, do = torch.from_numpy(pv).cuda(), torch.from_numpy(po).cuda()
    out = torch.empty((256, sum(t.shape[1] for t in tables)), device="cuda:0")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(_call_noalloc(lib, tables_dev, dv, do, out))
    assert lib.eb_noalloc_check_status(0, stream) == _lib.EB_OK
    bad = dv.clone()
    bad[3] = tables[0].shape[0] + 7  # an index past the first table's last row: skipped, and reported
    _lib.check(_call_noalloc(lib, tables_dev, bad, do, out))
    assert lib.eb_noalloc_check_status(0, stream) == _lib.EB_ERR_BAD_INPUT
    _lib.check(_call_noalloc(lib, tables_dev, dv, do, out))  # the next call starts from a clean status word
    assert lib.eb_noalloc_check_status(0, stream) == _lib.EB_OK
    # a call stages its descriptors through host memory that the next call overwrites: refused under capture
    graph = torch.cuda.CUDAGraph()
    scratch = torch.zeros(8, device="cuda:0")
    with torch.cuda.graph(graph):
        scratch.add_(1.0)
        rc = _call_noalloc(lib, tables_dev, dv, do, out)
    assert rc == _lib.EB_ERR_UNSUPPORTED and b"captured" in lib.eb_last_error()


def test_noalloc_two_host_threads_take_turns(lib):
    """Two host threads call the entry point on one GPU and one stream, each with its own model: the calls are
    serialised on the host (a per-device lock around staging, upload and launches) and run in order on the GPU."""
    import threading

    models = []
    for cfg_id, scale, batch in ((1, 0.1, 256), (2, 0.01, 300)):
        cfg, tables, values, offsets = small_model(cfg_id, scale, batch)
        pv, po = synth.pack_batch(values, offsets)
        models.append((tables, values, offsets, device_tables(tables), torch.from_numpy(pv).cuda(),
                       torch.from_numpy(po).cuda()))
    errors = []

    def worker(k):
        try:
            tables, values, offsets, tdev, dv, do = models[k]
            for _ in range(20):
                out = torch.full((do.shape[1] - 1, sum(t.shape[1] for t in tables)), float("nan"), device="cuda:0")
                _lib.check(_call_noalloc(lib, tdev, dv, do, out))
                torch.cuda.synchronize()
                check_against_oracle(out, tables, values, offsets, "f32")
        except Exception as e:  # noqa: BLE001 - reported by the main thread
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
