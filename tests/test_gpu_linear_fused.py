"""The one-launch decode linear (activation quantiser inside the GEMM kernel, M <= 16) through
dq_linear_w4a4_int4 against the two-launch path (dq_quant_act_int4 + dq_gemm_w4a4_int4) and the
oracle: outputs bit-identical to the former, < 1e-5 relative against the fp32 oracle epilogue."""
import pytest
import torch

from dualquant_b200 import _lib, ops, synthetic
from oracle import dq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _weights(N, K, seed):
    w = synthetic.make_w(N, K, seed)
    codes, sw = ops.quant_w_int4(w.to(DEV))
    return w, ops.pack_w_int4(codes, sw)


def _two_launch(x, a, pw, r, scale_fp16, out_dtype):
    codes, sx = ops.quant_act_int4(x, a, None, scale_fp16)
    return ops.gemm_w4a4_int4(codes, sx, pw, r, out_dtype=out_dtype)


@pytest.fixture(autouse=True)
def _fused_on():
    """The one-launch kernel is opt-in (dq_set_tuning("linear_fused", 1)); switch it on for these
    tests and restore the library defaults afterwards."""
    _lib.ensure_init(0)
    _lib.set_tuning("linear_fused", 1)
    yield
    for k, v in (("linear_fused", 0), ("fused_stages", 0), ("fused_split", 0), ("fused_extra_cta", 1)):
        _lib.set_tuning(k, v)


@pytest.mark.parametrize("M,N,K", [
    (1, 256, 512), (3, 384, 1024), (8, 4096, 4096), (16, 6144, 4096), (9, 3584, 4096),
    (16, 4096, 14336), (1, 4096, 14336), (5, 1000, 512), (16, 130, 128), (12, 2048, 2048),
    (16, 28672, 4096), (7, 768, 4096), (16, 512, 14336),
])
@pytest.mark.parametrize("scale_fp16", [False, True])
def test_fused_equals_two_launch_and_oracle(M, N, K, scale_fp16):
    w, pw = _weights(N, K, 3)
    r, c = synthetic.make_scales(N, K, 3)
    a = 1.0 / c
    x = synthetic.make_x(M, K, 10 + M)
    if M > 2:
        x[1] = 0  # an all-zero token
    xd, ad, rd = x.to(DEV), a.to(DEV), r.to(DEV)
    y = ops.linear_w4a4_int4(xd, ad, None, pw, rd, scale_fp16=scale_fp16)
    _lib.device_status(0)
    y2 = _two_launch(xd, ad, pw, rd, scale_fp16, torch.float32)
    assert torch.equal(y, y2)
    qx, sx, _ = O.quant_act_int4(x, a, None, scale_fp16)
    qw, sw = O.quant_w_int4(w)
    ref = O.dequant_matmul(qx, sx, qw, sw, r)
    err = (y.double().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 1e-5, err


@pytest.mark.parametrize("split", [1, 2, 4, 8])
@pytest.mark.parametrize("stages", [0, 2, 3])
def test_fused_forced_split_and_ring_depth(split, stages):
    M, N, K = 16, 1024, 4096
    w, pw = _weights(N, K, 4)
    r, c = synthetic.make_scales(N, K, 4)
    xd, ad, rd = synthetic.make_x(M, K, 4).to(DEV), (1.0 / c).to(DEV), r.to(DEV)
    y2 = _two_launch(xd, ad, pw, rd, True, torch.float32)
    _lib.set_tuning("fused_split", split)
    _lib.set_tuning("fused_stages", stages)
    y = ops.linear_w4a4_int4(xd, ad, None, pw, rd, scale_fp16=True)
    _lib.device_status(0)
    # a different split of K changes the order of the fp32 partial sums, not the integers
    assert (y - y2).abs().max() <= 2e-6 * y2.abs().max()
    _lib.set_tuning("linear_fused", 0)
    y3 = ops.linear_w4a4_int4(xd, ad, None, pw, rd, scale_fp16=True)
    assert torch.equal(y3, y2)


def test_fused_strided_rows_bf16_out_and_no_scales():
    M, N, K = 11, 640, 1024
    w, pw = _weights(N, K, 5)
    big = synthetic.make_x(M, 2 * K, 5).to(DEV)
    x = big[:, :K]  # row stride 2K
    y = ops.linear_w4a4_int4(x, None, None, pw, None, out_dtype=torch.bfloat16)
    y2 = _two_launch(x, None, pw, None, False, torch.bfloat16)
    _lib.device_status(0)
    assert y.dtype == torch.bfloat16 and torch.equal(y, y2)
    qx, sx, _ = O.quant_act_int4(x.cpu(), None, None, False)
    qw, sw = O.quant_w_int4(w)
    ref = O.dequant_matmul(qx, sx, qw, sw)
    assert ((y.double().cpu() - ref).abs().max() / ref.abs().max()) < 8e-3  # bf16 output rounding


def test_fused_rounding_boundaries_match_the_quantiser():
    """Rows built so that many x*a / s land on or next to half-integers: the in-kernel quantiser
    must take the same exact-division decisions as the stand-alone one."""
    M, N, K = 16, 256, 1024
    w, pw = _weights(N, K, 6)
    g = torch.Generator().manual_seed(6)
    halves = (torch.randint(-14, 15, (M, K), generator=g).float() * 0.5)
    halves[:, 0] = 7.0  # absmax 7 -> scale exactly 1
    x = halves.to(torch.bfloat16)
    x[3] = x[3] * 3.0  # absmax 21 -> scale 3: quotients k/2/3 with inexact reciprocals
    xd = x.to(DEV)
    y = ops.linear_w4a4_int4(xd, None, None, pw, None)
    y2 = _two_launch(xd, None, pw, None, False, torch.float32)
    _lib.device_status(0)
    assert torch.equal(y, y2)
    qx, sx, _ = O.quant_act_int4(x, None, None, False)
    qw, sw = O.quant_w_int4(w)
    ref = O.dequant_matmul(qx, sx, qw, sw)
    assert ((y.double().cpu() - ref).abs().max() / ref.abs().max()) < 1e-5
