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
    # a W4 checkpoint: the stored weight is the bf16 fake-quant of the raw one (group 128)
    w = O.dequant_w(*O.quant_w_int4(synthetic.make_w(N, K, 4))).to(torch.bfloat16)
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
    assert pl._packed is not None and pl._weight_on_grid is True  # the real int4 GEMM ran
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


def test_weight_off_the_int4_grid_keeps_the_reference_formulation():
    """The reference's PermLinear never quantises the weight (activations/perm_linear.py:136-141).
    A 16-bit weight (W16A4) must therefore not be pushed through the W4 GEMM: the layer runs
    fake-quantised activations into the wrapped layer's own F.linear, exactly the reference's
    formulation; force=True is the explicit opt-in to quantising the weight here."""
    K, N, M = 512, 256, 7
    lin = nn.Linear(K, N, bias=False).to(torch.bfloat16)
    lin.weight.data = synthetic.make_w(N, K, 5).clone()  # raw bf16 weight, not on the int4 grid
    fmt = formats.make_format("rtn_int4", block_size=-1)
    pl = PermLinear(lin.to(DEV), fmt)
    _, c = synthetic.make_scales(N, K, 5)
    pl.set_act_scale((1.0 / c).to(DEV))
    x = synthetic.make_x(M, K, 5).to(DEV)
    y = pl(x)
    assert pl._packed is None and pl._weight_on_grid is False
    assert torch.equal(y, pl.layer(pl._quantise_act(x)))
    xq, _, _ = O.quant_act_int4(x.cpu(), 1.0 / c, None, False)
    # opt-in: quantise the weight here and run the int4 GEMM
    assert pl.pack(force=True) is True
    y4 = pl(x)
    assert pl._packed is not None
    rel = (y4.float() - y.float()).abs().max() / y.float().abs().max()
    assert 1e-3 < rel < 0.2  # a different (W4) result, which is why it must be asked for


def test_fp32_inputs_are_quantised_from_fp32():
    """fp32 activations take the fp32 quantiser (the reference upcasts, perm_linear.py:119-125):
    codes equal the oracle's on the fp32 values, which differ from the codes of the bf16-rounded
    input on some elements."""
    K, N, M = 1024, 256, 5
    w = O.dequant_w(*O.quant_w_int4(synthetic.make_w(N, K, 6))).to(torch.bfloat16)
    lin = nn.Linear(K, N, bias=False).to(torch.bfloat16)
    lin.weight.data = w.clone()
    pl = PermLinear(lin.to(DEV), formats.make_format("rtn_int4", block_size=-1))
    _, c = synthetic.make_scales(N, K, 6)
    a = 1.0 / c
    pl.set_act_scale(a.to(DEV))
    g = torch.Generator().manual_seed(6)
    x = torch.randn(M, K, generator=g)  # fp32 values that are not bf16-representable
    y = pl(x.to(DEV))
    qx, sx, _ = O.quant_act_int4(x, a, None, False)
    qw, sw = O.quant_w_int4(w)
    ref = O.dequant_matmul(qx, sx, qw, sw)
    err = (y.double().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 8e-3  # bf16 output rounding only
    from dualquant_b200 import ops
    codes, s_dev = ops.quant_act_int4(x.to(DEV), a.to(DEV), None, False)
    assert torch.equal(codes.cpu(), qx) and torch.equal(s_dev.cpu(), sx)
    qx_bf16, _, _ = O.quant_act_int4(x.to(torch.bfloat16), a, None, False)
    assert not torch.equal(qx_bf16, qx)


@pytest.mark.parametrize("name", ["mxfp4", "nvfp4"])
def test_fp4_forward_close_to_fakequant_reference(name):
    # PermLinear with an FP4 activation format and a weight already on that format's grid runs the
    # packed FP4 GEMM; compare with the fake-quant formulation (cast both operands, fp64 matmul)
    # the reference computes
    K, N, M = 512, 256, 9
    w = synthetic.make_w(N, K, 8)
    if name == "mxfp4":
        w = O.quant_mxfp4(w.float())[2].to(torch.bfloat16)  # exact in bf16
    else:
        w = O.quant_nvfp4(w.float(), float((w.float().abs().max() / 2688.0).item()))[3].to(torch.bfloat16)
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
    assert pl._packed_fp4 is not None and pl._weight_on_grid_fp4 is True
    x32 = x.float() * a
    if name == "mxfp4":
        xd, wd = O.quant_mxfp4(x32)[2], O.quant_mxfp4(w.float())[2]
    else:
        xd = O.quant_nvfp4(x32)[3]
        wd = O.quant_nvfp4(w.float(), float((w.float().abs().max() / 2688.0).item()))[3]
    ref = xd.double() @ wd.double().T
    assert ((y - ref).abs().max() / ref.abs().max()).item() < 8e-3  # bf16 output rounding


def test_bf16_arithmetic_branch_bit_exact_against_the_reference(golden):
    """No activation scale, no Hadamard, bf16 input: the reference quantises in bf16 arithmetic
    (activations/perm_linear.py:131-133).  De-quantised activations equal the reference's tensor bit
    for bit; codes and scales equal the oracle's; the int4 GEMM output agrees to bf16 accuracy."""
    from dualquant_b200 import ops

    w = _bf16(golden["perm_noscale_w_bf16"])
    lin = nn.Linear(w.shape[1], w.shape[0], bias=False).to(torch.bfloat16)
    lin.weight.data = w.clone()
    pl = PermLinear(lin.to(DEV), formats.make_format("rtn_int4", block_size=-1))
    x = _bf16(golden["perm_noscale_x"])
    xq = pl._quantise_act(x.to(DEV)).cpu()
    assert torch.equal(xq, _bf16(golden["perm_noscale_xq_bf16"]))
    q, s, _ = O.quant_act_int4_bf16_arith(x)
    codes, sx = ops.quant_act_int4(x.to(DEV), None, None, bf16_arith=True)
    assert torch.equal(codes.cpu(), q) and torch.equal(sx.cpu(), s)
    # the format object's cast on a bf16 tensor takes the same branch
    f = formats.make_format("rtn_int4", block_size=-1)
    assert torch.equal(f.cast(x.to(DEV)).cpu(), _bf16(golden["perm_noscale_xq_bf16"]))
    y = pl(x.to(DEV)).float().cpu()
    assert pl._packed is not None
    ref = _bf16(golden["perm_noscale_y_bf16"]).float()
    assert (y - ref).abs().max() / ref.abs().max() < 2e-2
    # exact integer sums of exactly these codes
    qw, sw = O.quant_w_int4(w)
    exact = O.dequant_matmul(q, s, qw, sw)
    assert ((y.double() - exact).abs().max() / exact.abs().max()) < 8e-3
