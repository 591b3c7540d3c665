"""GPU parity against the reference itself: its device templates (compiled from the reference checkout into
oracle/_ref/libref_kernels.so by oracle/build_ref.sh) and the golden fixtures made with its Python checker."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from recflex_b200.rec_modules import FeatEmbed, FeatProcessEmbed, Schedule
from tests.helpers import TOL, all_schedules, device_tables, small_model, to_device
from tests.test_oracle import CASES, load_case

pytestmark = pytest.mark.gpu

REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                       "libref_kernels.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_LIB):
        if os.environ.get("RECFLEX_REF"):
            pytest.fail("a RecFlex checkout is configured ($RECFLEX_REF) but oracle/_ref/libref_kernels.so was not "
                        "built: run oracle/build_ref.sh")
        pytest.skip("oracle/_ref/libref_kernels.so was not built (needs the reference checkout: oracle/build_ref.sh)")
    lib = C.CDLL(REF_LIB)
    lib.ref_pool_feature.restype = C.c_int
    lib.ref_pool_feature.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                     C.c_int, C.c_void_p]
    lib.ref_onehot_feature.restype = C.c_int
    lib.ref_onehot_feature.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    return lib


def reference_kernels_output(ref, kind, tables_dev, values_dev, offsets_dev, onehot_feats=()):
    """Run the reference's ws (kind 0) / obms (kind 1) template per feature; one-hot features through its
    onehot::GatherSegments.  Returns [batch, sum(dim)]."""
    batch = offsets_dev[0].numel() - 1
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    cols = []
    for f, (t, v, o) in enumerate(zip(tables_dev, values_dev, offsets_dev)):
        out = torch.full((batch, t.shape[1]), float("nan"), device=t.device)
        if f in onehot_feats:
            rc = ref.ref_onehot_feature(t.shape[1], t.data_ptr(), v.data_ptr(), out.data_ptr(), v.numel(), stream)
        else:
            rc = ref.ref_pool_feature(kind, t.shape[1], t.data_ptr(), v.data_ptr(), o.data_ptr(), out.data_ptr(),
                                      v.numel(), batch, stream)
        assert rc == 0, f"reference harness returned {rc} for feature {f} (dim {t.shape[1]})"
        cols.append(out)
    torch.cuda.synchronize()
    return torch.cat(cols, dim=1)


@pytest.mark.parametrize("cfg_id,scale,batch", [(1, 1.0, 256), (2, 0.02, 1024), (5, 0.02, 512)])
@pytest.mark.parametrize("ref_kind", [0, 1])
def test_matches_reference_device_templates(ref, cfg_id, scale, batch, ref_kind):
    cfg, tables, values, offsets = small_model(cfg_id, scale, batch)
    tables_dev = device_tables(tables)
    dv, do = to_device(values), to_device(offsets)
    onehot = {f for f, fs in enumerate(cfg.features) if fs.length == "onehot"}
    expect = reference_kernels_output(ref, ref_kind, tables_dev, dv, do, onehot_feats=onehot)
    assert not torch.isnan(expect).any()
    mod = FeatEmbed("cuda:0", embed_tables=tables_dev)
    for kind in ("stream", "pipe", "flat", "warp", "group"):
        mod.set_schedules(all_schedules(kind, 4, len(tables)))
        out = mod(dv, do)
        mod.check_status()
        torch.testing.assert_close(out, expect, **TOL["f32"])


@pytest.mark.parametrize("name", CASES)
def test_golden_fixtures_through_the_text_front_end(name):
    tables, raw, expect = load_case(name)
    model = FeatProcessEmbed(None, 0, embed_tables=device_tables(tables))
    tag = "f16" if tables[0].dtype == np.float16 else "f32"
    for kind in ("stream", "pipe", "flat", "warp", "group"):
        model.embed_layer.set_schedules(all_schedules(kind, 2, len(tables)))
        out = model(raw)
        np.testing.assert_allclose(out.cpu().numpy(), expect, **TOL[tag])
