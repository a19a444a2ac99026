"""A16W4 (16-bit activations x int4 weights on tcgen05 kind::f16) through the C ABI.  The checks are
the reference's own (vendor/dualscale_kernel_benchmark/fused_dual_scale_kernel.py:269-308: seed 42,
four shapes, mean relative error below 1 % against (x * beta) @ dequant(W)^T) plus a tight bound
against the restatement of this kernel's arithmetic (both operands rounded to fp16, fp64 sum)."""
import pytest
import torch
import torch.nn as nn

from dualquant_b200 import _lib, formats, ops, synthetic
from dualquant_b200.activations import PermLinear
from oracle import dq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _restatement(x, a, qw, sw, r=None):
    """fp16(x * a) @ fp16(code * scale)^T in fp64, times r."""
    xs = x.float() * a.float() if a is not None else x.float()
    xs = xs.clamp(-65504.0, 65504.0).to(torch.float16)
    N, K = qw.shape
    w = (qw.float().reshape(N, K // 128, 128) * sw.float().reshape(N, K // 128, 1)).to(torch.float16).reshape(N, K)
    y = xs.double() @ w.double().T
    return y if r is None else y * r.double().reshape(1, N)


# the reference's four check shapes (M, N, K), its seed and its tolerance
@pytest.mark.parametrize("M,N,K", [(4, 64, 128), (16, 256, 256), (1, 4096, 4096), (128, 4096, 4096)])
def test_reference_check_shapes(M, N, K):
    torch.manual_seed(42)
    W = torch.randn(N, K)
    x = torch.randn(M, K).to(torch.bfloat16)
    beta = (torch.rand(K) * 0.4 + 0.8).to(torch.bfloat16)
    qw, sw = O.quant_w_int4(W.to(torch.bfloat16))
    pw = ops.pack_w_int4(qw.to(DEV), sw.to(DEV))
    y = ops.linear_a16w4(x.to(DEV), beta.float().to(DEV), pw).float().cpu()
    _lib.device_status(0)
    w_dq = O.dequant_w(qw, sw)                       # dequant_int4_reference
    y_ref = (x.float() * beta.float()) @ w_dq.T      # the reference's unfused formulation
    rel = ((y - y_ref).abs() / (y_ref.abs() + 1e-6)).mean().item()
    assert rel < 0.01, rel
    tight = _restatement(x, beta.float(), qw, sw)
    err = ((y.double() - tight).abs().max() / tight.abs().max()).item()
    assert err < 8e-3, err  # bf16 output rounding of an fp32 accumulation


@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (16, 384, 1024), (32, 1000, 512), (33, 512, 4096),
                                   (128, 640, 2048), (300, 4096, 4096), (2048, 4096, 4096), (64, 4096, 14336)])
def test_a16w4_matches_restatement_fp32_out(M, N, K):
    w = synthetic.make_w(N, K, 17)
    qw, sw = O.quant_w_int4(w)
    pw = ops.pack_w_int4(qw.to(DEV), sw.to(DEV))
    r, c = synthetic.make_scales(N, K, 17)
    a = 1.0 / c
    x = synthetic.make_x(M, K, 17 + M)
    y = ops.linear_a16w4(x.to(DEV), a.to(DEV), pw, r.to(DEV), out_dtype=torch.float32)
    _lib.device_status(0)
    rows = torch.arange(M) if M <= 64 else torch.randperm(M, generator=torch.Generator().manual_seed(1))[:64]
    ref = _restatement(x[rows], a, qw, sw, r)
    got = y.cpu()[rows].double()
    err = ((got - ref).abs().max() / ref.abs().max()).item()
    assert err < 1e-4, err  # exact fp16 products, fp32 accumulation on the tensor cores
    # without the column scale
    y2 = ops.linear_a16w4(x.to(DEV), None, pw, None, out_dtype=torch.float32)
    ref2 = _restatement(x[rows], None, qw, sw)
    assert ((y2.cpu()[rows].double() - ref2).abs().max() / ref2.abs().max()).item() < 1e-4
    _lib.device_status(0)


def test_perm_linear_without_activation_cast_runs_a16w4():
    """act_quant_enabled = False on a W4 layer: the reference computes bf16(x * act_scale) @ W^T
    (activations/perm_linear.py:108-141); here the packed int4 weight is used on the bf16 tensor
    cores instead of the layer's 16-bit copy."""
    K, N, M = 1024, 512, 20
    w = O.dequant_w(*O.quant_w_int4(synthetic.make_w(N, K, 19))).to(torch.bfloat16)
    lin = nn.Linear(K, N, bias=False).to(torch.bfloat16)
    lin.weight.data = w.clone()
    pl = PermLinear(lin.to(DEV), formats.make_format("rtn_int4", block_size=-1))
    _, c = synthetic.make_scales(N, K, 19)
    pl.set_act_scale((1.0 / c).to(DEV))
    pl.set_act_quant_enabled(False)
    x = synthetic.make_x(M, K, 19).to(DEV)
    y = pl(x)
    assert pl._packed is not None and y.dtype == torch.bfloat16
    ref = pl.layer(pl._quantise_act(x))  # the reference's formulation on the 16-bit weight
    err = ((y.float() - ref.float()).abs().max() / ref.float().abs().max()).item()
    assert err < 2e-2, err  # bf16 rounding of the output; the reference rounds x * a to bf16, this path to fp16
