"""DualQuant's offline scale search (block coordinate descent) and final block quantisation,
batched over the column blocks of a weight (dualquant_b200/bcd.py), against vectors recorded from
the reference's wrap_dualquant_layer (layer_wrapper_dualquant.py:423-533, CPU, block after block).

Floating point: the batched form sums in another order than the reference's per-block loop, so the
bar is a tolerance - scales and stored weights within 2e-6 relative (measured 4e-7; the E8M0 and
column-only configurations come out bit-identical)."""
import os

import numpy as np
import pytest
import torch

from dualquant_b200 import bcd

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.npz")
CFGS = {
    "iter15": dict(scale_option="row_column", row_init="max_abs", col_init="l1_norm", num_iter=15, scale_format="none"),
    "e4m3": dict(scale_option="row_column", row_init="max_abs", col_init="l2_norm", num_iter=5, scale_format="e4m3"),
    "e8m0": dict(scale_option="row_column", row_init="max_abs", col_init="l1_norm", num_iter=5, scale_format="e8m0"),
    "colonly": dict(scale_option="only_column", row_init="max_abs", col_init="l1_norm", num_iter=5, scale_format="none"),
}
RTOL = 2e-6


@pytest.fixture(scope="module")
def vec():
    return np.load(GOLDEN)


def _check(mat_q, cs, vec, tag):
    gm = torch.from_numpy(vec[f"bcd_{tag}_matq"])
    gc = torch.from_numpy(vec[f"bcd_{tag}_colscales"])
    assert mat_q.shape == gm.shape and cs.shape == gc.shape
    assert ((mat_q.cpu() - gm).abs().max() / gm.abs().max()).item() < RTOL
    assert ((cs.cpu() - gc).abs() / gc.abs()).max().item() < RTOL


@pytest.mark.parametrize("tag", sorted(CFGS))
def test_matches_reference_on_cpu(vec, tag):
    W = torch.from_numpy(vec["bcd_w"])
    mat_q, cs = bcd.dualquant_weight(W, block_size=128, **CFGS[tag])
    _check(mat_q, cs, vec, tag)
    if tag in ("e8m0", "colonly"):  # no unrounded row scale in the loop: bit-identical
        assert torch.equal(mat_q, torch.from_numpy(vec[f"bcd_{tag}_matq"]))


def test_wrap_dualquant_layer_is_a_drop_in(vec):
    W = torch.from_numpy(vec["bcd_w"])
    cfg = dict(num_splits=1, block_size=128, dualquant_to_element_tensor=True, **CFGS["e8m0"])
    lin = torch.nn.Linear(256, 96, bias=False)
    lin.weight.data.copy_(W)
    cs = bcd.wrap_dualquant_layer(lin, cfg, "rtn_int4", act_quant_flag=True)
    _check(lin.weight.data, cs, vec, "e8m0")
    # without activation quantisation the column scales are folded back into the stored weight
    lin2 = torch.nn.Linear(256, 96, bias=False)
    lin2.weight.data.copy_(W)
    assert bcd.wrap_dualquant_layer(lin2, cfg, "rtn_int4", act_quant_flag=False) is None
    assert torch.allclose(lin2.weight.data, lin.weight.data * cs.unsqueeze(0), rtol=1e-6, atol=0)


def test_search_lowers_the_reconstruction_error(vec):
    """What the search is for: W ~ mat_q * column_scales is closer to W than plain group-RTN."""
    W = torch.from_numpy(vec["bcd_w"])
    W3 = W.reshape(96, 2, 128)
    s = W3.abs().amax(dim=-1, keepdim=True) / 7.0
    rtn = ((W3 / s).round().clamp(-8, 7) * s).reshape(96, 256)
    mat_q, cs = bcd.dualquant_weight(W, block_size=128, **CFGS["iter15"])
    assert ((mat_q * cs - W) ** 2).mean() < 0.9 * ((rtn - W) ** 2).mean()


def test_unsupported_options_say_so():
    W = torch.randn(8, 128)
    with pytest.raises(NotImplementedError):
        bcd.dualquant_weight(W, quant_method="nvfp4")
    with pytest.raises(NotImplementedError):
        bcd.dualquant_weight(W, scale_format="e5m3")
    with pytest.raises(ValueError):
        bcd.dualquant_weight(W, block_size=96)
    with pytest.raises(ValueError):
        bcd.dualquant_weight(W, scale_option="both")


@pytest.mark.gpu
@pytest.mark.parametrize("tag", sorted(CFGS))
def test_matches_reference_on_the_gpu_and_packs(vec, tag):
    """The same search on the device, then DualQuant's outputs -> packed int4 artefact -> W4A4 linear:
    the stored weight lies on the int4 group grid, so packing it loses nothing."""
    from dualquant_b200 import _lib, ops, wrap
    from oracle import dq_oracle as O

    dev = "cuda:0"
    W = torch.from_numpy(vec["bcd_w"])
    mat_q, cs = bcd.dualquant_weight(W.to(dev), block_size=128, **CFGS[tag])
    _check(mat_q, cs, vec, tag)
    pw, a = wrap.pack_from_dualquant(mat_q, cs)
    x = torch.randn(24, 256, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    y = ops.linear_w4a4_int4(x.to(dev), a, None, pw, None, scale_fp16=False)
    _lib.device_status(0)
    qx, sx, _ = O.quant_act_int4(x, cs.cpu(), None, False)
    qw, sw = O.quant_w_int4(mat_q.cpu().to(torch.bfloat16))
    ref = O.dequant_matmul(qx, sx, qw, sw, None)
    assert ((y.cpu().double() - ref).abs().max() / ref.abs().max()).item() < 1e-5
    # the artefact's codes x fp16 group scales reproduce the stored weight to its bf16 storage
    # rounding (2^-8 relative; the reference keeps mat_q in the layer's bf16 weight as well)
    back = O.dequant_w(qw, sw)
    assert ((back - mat_q.cpu()).abs().max() / mat_q.abs().max().cpu()).item() < 6e-3


@pytest.mark.gpu
def test_full_size_layer_on_the_gpu():
    """A 4096 x 4096 weight (32 column blocks searched at once): finite scales, lower error than
    group-RTN, and every block equal to the same block searched on its own."""
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(5)
    W = torch.randn(4096, 4096, generator=g, device=dev) * 0.02
    W[:, torch.randperm(4096, generator=g, device=dev)[:40]] *= 10
    cfg = CFGS["e8m0"]
    mat_q, cs = bcd.dualquant_weight(W, block_size=128, **cfg)
    assert torch.isfinite(mat_q).all() and torch.isfinite(cs).all()
    W3 = W.reshape(4096, 32, 128)
    s = W3.abs().amax(dim=-1, keepdim=True) / 7.0
    rtn = ((W3 / s).round().clamp(-8, 7) * s).reshape(4096, 4096)
    assert ((mat_q * cs - W) ** 2).mean() < ((rtn - W) ** 2).mean()
    for b in (0, 17, 31):
        mq_b, cs_b = bcd.dualquant_weight(W[:, b * 128:(b + 1) * 128].contiguous(), block_size=128, **cfg)
        assert torch.allclose(mq_b, mat_q[:, b * 128:(b + 1) * 128], rtol=1e-5, atol=1e-9)
        assert torch.allclose(cs_b, cs[b * 128:(b + 1) * 128], rtol=1e-5, atol=0)
