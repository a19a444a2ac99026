"""PermLinear / FormatSpec drop-ins on the GPU against vectors recorded from the reference's own
PermLinear (tests/golden/make_golden.py) and against the oracle."""
import pytest
import torch
import torch.nn as nn

from dualquant_b200 import formats, quarot, synthetic
from dualquant_b200.activations import PermLinear
from oracle import dq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bf16(arr):
    return torch.from_numpy(arr.copy()).view(torch.bfloat16)


def _module(golden, tag):
    w = _bf16(golden[f"perm_{tag}_w_bf16"])
    lin = nn.Linear(w.shape[1], w.shape[0], bias=False).to(torch.bfloat16)
    lin.weight.data = w.clone()
    pl = PermLinear(lin.to(DEV), formats.make_format("rtn_int4", block_size=-1))
    pl.set_act_scale(torch.from_numpy(golden[f"perm_{tag}_a"]).to(DEV))
    return pl, _bf16(golden[f"perm_{tag}_x"]).to(DEV)


@pytest.mark.parametrize("tag", ["plain", "full", "partial"])
def test_forward_against_reference_outputs(golden, tag):
    pl, x = _module(golden, tag)
    K = x.shape[1]
    if tag == "full":
        pl.online_full_had = True
        pl.had_K, pl.K = quarot.get_hadK(K)
    elif tag == "partial":
        pl.online_partial_had = True
        pl.had_K, pl.K = quarot.get_hadK(K // 8)
        pl.had_dim = 8
    y = pl(x).float().cpu()
    ref = _bf16(golden[f"perm_{tag}_y_bf16"]).float()
    # the reference rounds both de-quantised operands and the output to bf16 and keeps fp32 weight
    # scales; the int4 path keeps exact integers and fp16 group scales: agreement to bf16 accuracy
    err = (y - ref).abs().max() / ref.abs().max()
    assert err < 2e-2, err
    sqnr = 10 * torch.log10(ref.pow(2).sum() / (y - ref).pow(2).sum())
    assert sqnr > 35
    # the de-quantised activations themselves (what the reference feeds its F.linear)
    xq = pl._quantise_act(x).float().cpu()
    xq_ref = _bf16(golden[f"perm_{tag}_xq_bf16"]).float()
    if tag == "full":
        step = xq_ref.abs().amax(dim=1, keepdim=True) / 7
        assert ((xq - xq_ref).abs() > 1e-3 * step).float().mean() < 2e-3
    else:
        assert torch.equal(xq, xq_ref)


def test_forward_matches_oracle_and_handles_leading_dims():
    K, N = 1024, 384
    w = synthetic.make_w(N, K, 4)
    lin = nn.Linear(K, N, bias=True).to(torch.bfloat16)
    lin.weight.data = w.clone()
    pl = PermLinear(lin.to(DEV), formats.make_format("rtn_int4", block_size=-1))
    _, c = synthetic.make_scales(N, K, 4)
    a = 1.0 / c
    pl.set_act_scale(a)
    pl = pl.to(DEV)
    x = synthetic.make_x(6, K, 4).reshape(2, 3, K)
    y = pl(x.to(DEV))
    assert y.shape == (2, 3, N) and y.dtype == torch.bfloat16
    qx, sx, _ = O.quant_act_int4(x.reshape(6, K), a, None, False)
    qw, sw = O.quant_w_int4(w)
    ref = O.dequant_matmul(qx, sx, qw, sw) + lin.bias.detach().double().cpu()
    err = (y.reshape(6, N).double().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 8e-3  # bf16 output rounding


def test_quantize_bmm_input_and_disabled_quant():
    K, N = 256, 128
    lin = nn.Linear(K, N, bias=False).to(torch.bfloat16).to(DEV)
    fmt = formats.make_format("rtn_int4", block_size=-1)
    pl = PermLinear(lin, fmt, quantize_bmm_input=True)
    x = synthetic.make_x(4, K, 2).to(DEV)
    y = pl(x)
    # every output row lies on its own 15-level grid
    for row in y.float():
        s = row.abs().max() / 7
        q = row / s
        assert torch.allclose(q, q.round(), atol=2e-2)
    pl2 = PermLinear(lin, fmt)
    pl2.set_act_quant_enabled(False)
    assert torch.equal(pl2(x), lin(x))  # pass-through when nothing is configured


def test_format_cast_matches_reference(golden):
    f = formats.make_format("rtn_int4", block_size=-1)
    x32 = torch.from_numpy(golden["cast_in"]).to(DEV)
    assert torch.equal(f.cast(x32).cpu(), torch.from_numpy(golden["cast_out"]))
    fw = formats.make_format("rtn_int4", block_size=128)
    w = torch.from_numpy(golden["wcast_in"]).to(DEV)
    assert torch.equal(fw.cast(w).cpu(), torch.from_numpy(golden["wcast_out"]))


@pytest.mark.parametrize("name", ["mxfp4", "nvfp4"])
def test_fp4_forward_close_to_fakequant_reference(name):
    # PermLinear with an FP4 activation format runs the packed FP4 GEMM; compare with the
    # fake-quant formulation (cast both operands, fp64 matmul) the reference computes
    K, N, M = 512, 256, 9
    w = synthetic.make_w(N, K, 8)
    lin = nn.Linear(K, N, bias=False).to(torch.bfloat16)
    lin.weight.data = w.clone()
    fmt = formats.make_format(name)
    pl = PermLinear(lin.to(DEV), fmt)
    _, c = synthetic.make_scales(N, K, 8)
    a = 1.0 / c
    pl.set_act_scale(a)
    pl = pl.to(DEV)
    x = synthetic.make_x(M, K, 8)
    y = pl(x.to(DEV)).double().cpu()
    x32 = x.float() * a
    if name == "mxfp4":
        xd, wd = O.quant_mxfp4(x32)[2], O.quant_mxfp4(w.float())[2]
    else:
        xd = O.quant_nvfp4(x32)[3]
        wd = O.quant_nvfp4(w.float(), float((w.float().abs().max() / 2688.0).item()))[3]
    ref = xd.double() @ wd.double().T
    assert ((y - ref).abs().max() / ref.abs().max()).item() < 8e-3  # bf16 output rounding
