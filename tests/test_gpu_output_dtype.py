"""GPU: the narrow output modes (bfloat16 / binary16 rows) and the end-to-end model that uses them."""
import numpy as np
import pytest
import torch

from oracle import oracle
from recflex_b200.rec_modules import FeatEmbed, RecomModel, Schedule
from tests.helpers import all_schedules, device_tables, small_model, to_device

pytestmark = pytest.mark.gpu

KINDS = ["group", "warp", "flat", "stream", "pipe"]


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cfg_id,scale,batch", [(3, 2e-4, 700), (2, 0.01, 515)])
def test_narrow_output_is_the_rounded_fp32_output(kind, dtype, cfg_id, scale, batch):
    """Narrow rows must be the fp32 rows rounded to nearest even: bit-exact for every bag that one slot pooled in one
    go (all of them under group / warp / flat; under stream / pipe all but the bags cut by a piece boundary, whose
    first part is rounded once more), exactly 0 for empty bags."""
    cfg, tables, values, offsets = small_model(cfg_id, scale, batch)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    mod.set_schedules(all_schedules(kind, 4, len(tables)))
    dv, do = to_device(values), to_device(offsets)
    ref = mod(dv, do)
    mod.set_output_dtype(dtype)
    out = mod(dv, do)
    mod.check_status()
    assert out.dtype == dtype and out.shape == ref.shape
    rounded = ref.to(dtype)
    if kind in ("group", "warp", "flat"):
        assert torch.equal(out, rounded)
    else:
        same = (out == rounded).float().mean().item()
        assert same > 0.9, f"only {same:.3f} of the cells equal the rounded fp32 result"
        mags = torch.from_numpy(oracle.pool([np.abs(t) for t in tables], values, offsets, acc64=True)).cuda()
        ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
        assert ((out.float() - ref).abs() <= 2 * ulp * mags + 1e-7).all()
    col = 0
    for t, o in zip(tables, offsets):
        empty = torch.from_numpy(np.nonzero(np.diff(o) == 0)[0]).cuda()
        assert (out[empty, col:col + t.shape[1]] == 0).all()
        col += t.shape[1]
    # odd leading dimension and column offset: the scalar store path
    wide = torch.zeros((batch, mod.output_units + 3), dtype=dtype, device="cuda:0")
    mod(dv, do, out=wide[:, 1:1 + mod.output_units])
    assert torch.equal(wide[:, 1:1 + mod.output_units], out)
    mod.set_output_dtype(torch.float32)
    assert torch.equal(mod(dv, do), ref)


def test_narrow_output_through_the_host_and_packed_calls():
    from recflex_b200 import synth

    cfg, tables, values, offsets = small_model(1, 0.1, 256)
    mod = FeatEmbed("cuda:0", embed_tables=device_tables(tables))
    pv, po = synth.pack_batch(values, offsets)
    ref = mod.forward_packed(torch.from_numpy(pv).cuda(), torch.from_numpy(po).cuda())
    mod.set_output_dtype(torch.bfloat16)
    host = mod.forward_host(torch.from_numpy(pv).pin_memory(), torch.from_numpy(po).pin_memory())
    torch.cuda.synchronize()
    assert host.dtype == torch.bfloat16
    # one rounding to 8 significant bits, a second one for the first part of a bag cut by a piece boundary
    mags = torch.from_numpy(oracle.pool([np.abs(t) for t in tables], values, offsets, acc64=True))
    assert ((host.float() - ref.cpu()).abs() <= 2 * 2.0 ** -8 * mags + 1e-7).all()


@pytest.mark.parametrize("mlp_dtype", [torch.float32, torch.bfloat16])
def test_recom_model_matches_oracle_pooling_plus_the_same_mlp(mlp_dtype):
    """RecomModel = fused embedding -> MLP -> sigmoid (reference: RecFlex/rec_modules.py:143-179, driven by
    examples/end_to_end.py:39-51 with layers [1024, 256, 128]).  Expected: the oracle's pooled rows through the same
    weights in float64 on the CPU."""
    cfg, tables, values, offsets = small_model(2, 0.01, 300)
    torch.manual_seed(0)
    model = RecomModel([1024, 256, 128], "cuda:0", embed_tables=device_tables(tables), mlp_dtype=mlp_dtype)
    assert model.embed_layer.output_units == sum(t.shape[1] for t in tables)
    out = model(to_device(values), to_device(offsets))
    model.embed_layer.check_status()
    assert out.shape == (300, 1) and out.dtype == mlp_dtype
    x = torch.from_numpy(oracle.pool(tables, values, offsets, acc64=True)).double()
    for layer in model.mlp:
        if isinstance(layer, torch.nn.Linear):
            x = x @ layer.weight.detach().double().cpu().T + layer.bias.detach().double().cpu()
        elif isinstance(layer, torch.nn.ReLU):
            x = torch.relu(x)
        else:
            x = torch.sigmoid(x)
    # fp32: cuBLAS may use TF32-free fp32 accumulation in another order; bf16: 8-bit significands through four layers
    tol = dict(rtol=1e-4, atol=1e-5) if mlp_dtype == torch.float32 else dict(rtol=0, atol=2e-2)
    torch.testing.assert_close(out.double().cpu(), x, **tol)
