"""Producer / consumer fusions either side of the int4 GEMM: the residual connection added in the
GEMM epilogue and the one-pass bf16 fake-quantisation of a linear's output (PermLinear's
quantize_bmm_input step, activations/perm_linear.py:139-140)."""
import pytest
import torch
import torch.nn as nn

from dualquant_b200 import _lib, formats, ops, synthetic
from dualquant_b200.activations import PermLinear
from oracle import dq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# M = 1 / 16: decode kernel; 48: tcgen05 kernel with weights through tensor memory; 160: tcgen05
# kernel with int8 weight tiles in shared memory.  (256, 4096): split-K over a cluster at small M.
@pytest.mark.parametrize("M", [1, 16, 48, 160])
@pytest.mark.parametrize("N,K", [(384, 512), (256, 4096)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_residual_in_the_epilogue_equals_a_separate_add(M, N, K, dtype):
    w = synthetic.make_w(N, K, 9)
    codes_w, sw = ops.quant_w_int4(w.to(DEV))
    pw = ops.pack_w_int4(codes_w, sw)
    r, c = synthetic.make_scales(N, K, 9)
    x = synthetic.make_x(M, K, 9 + M)
    codes, sx = ops.quant_act_int4(x.to(DEV), (1.0 / c).to(DEV), None, False)
    g = torch.Generator().manual_seed(M)
    res = torch.randn(M, N, generator=g).to(dtype).to(DEV)
    plain = ops.gemm_w4a4_int4(codes, sx, pw, r.to(DEV), out_dtype=dtype)
    fused = ops.gemm_w4a4_int4(codes, sx, pw, r.to(DEV), residual=res)
    _lib.device_status(0)
    assert fused.dtype == dtype
    assert torch.equal(fused, plain + res)  # bf16: bf16(bf16(linear) + residual); fp32: one fp32 add
    # in place: the residual buffer is also the output
    buf = res.clone()
    ops.gemm_w4a4_int4(codes, sx, pw, r.to(DEV), out=buf, residual=buf)
    _lib.device_status(0)
    assert torch.equal(buf, fused)


@pytest.mark.parametrize("M,K", [(1, 128), (7, 4096), (33, 6144), (5, 14336)])
def test_bf16_fakequant_matches_cast_of_the_fp32_tensor(M, K):
    g = torch.Generator().manual_seed(K + M)
    y = (torch.randn(M, K, generator=g) * 3).to(torch.bfloat16)
    if M > 2:
        y[1] = 0
    got = ops.fakequant_act_int4_bf16(y.to(DEV)).cpu()
    q, s, _ = O.quant_act_int4(y.float(), None, None, False)
    ref = (q.float() * s.reshape(-1, 1)).to(torch.bfloat16)
    assert torch.equal(got, ref)
    # the format object's cast on the fp32 copy, rounded to bf16, is the same tensor
    f = formats.make_format("rtn_int4", block_size=-1)
    assert torch.equal(f.cast(y.float().to(DEV)).to(torch.bfloat16).cpu(), got)
    _lib.device_status(0)


def test_perm_linear_quantize_bmm_input_uses_the_same_values():
    K, N, M = 512, 256, 6
    w = O.dequant_w(*O.quant_w_int4(synthetic.make_w(N, K, 12))).to(torch.bfloat16)
    lin = nn.Linear(K, N, bias=False).to(torch.bfloat16)
    lin.weight.data = w.clone()
    fmt = formats.make_format("rtn_int4", block_size=-1)
    plain = PermLinear(lin.to(DEV), fmt)
    quant = PermLinear(lin, fmt, quantize_bmm_input=True)
    x = synthetic.make_x(M, K, 12).to(DEV)
    y = plain(x)
    yq = quant(x)
    assert torch.equal(yq, fmt.cast(y.float()).to(torch.bfloat16))
