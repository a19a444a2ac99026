"""The per-(token, K tile) activation-scale variant (the arithmetic of the reference's fused W4A4
Triton kernel, ablation/real_int4_kernel/fused_w4a4_kernel.py:93-119, with groups of 128) through
the C ABI against the oracle: codes and scales bit-exact, outputs within 1e-5 of the fp32 oracle
epilogue."""
import pytest
import torch

from dualquant_b200 import _lib, ops, synthetic
from oracle import dq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("M,K", [(1, 128), (5, 1024), (40, 4096), (3, 14336)])
@pytest.mark.parametrize("round_away", [False, True])
@pytest.mark.parametrize("scale_fp16", [False, True])
def test_grouped_quantiser_bit_exact(M, K, round_away, scale_fp16):
    x = synthetic.make_x(M, K, 5 + M)
    if M > 2:
        x[1] = 0
        x[2, 128:256] = 0  # one all-zero tile
    # tiles whose maximum is 7 (scale 1) with halves as quotients: the two rounding modes differ
    x[0, :128] = (torch.arange(128) % 15 - 7).float().mul(0.5).to(torch.bfloat16)
    x[0, 0] = 7.0
    _, c = synthetic.make_scales(8, K, 3)
    a = 1.0 / c
    for av in (None, a):
        q, s = O.quant_act_int4_grouped(x, av, 128, scale_fp16, round_away)
        codes, sxg = ops.quant_act_int4_grouped(x.to(DEV), None if av is None else av.to(DEV), scale_fp16, round_away)
        _lib.device_status(0)
        assert torch.equal(sxg.cpu().T.contiguous(), s)
        assert torch.equal(codes.cpu(), q)
    q_even, _ = O.quant_act_int4_grouped(x, None, 128, scale_fp16, False)
    q_away, _ = O.quant_act_int4_grouped(x, None, 128, scale_fp16, True)
    assert not torch.equal(q_even[0, :128], q_away[0, :128])


# M <= 16: decode kernel; above: tcgen05 kernel with the weights through tensor memory (token tiles
# 32 / 64 / 128); (256, 4096): split-K over a cluster
@pytest.mark.parametrize("M", [1, 8, 16, 24, 64, 100, 300])
@pytest.mark.parametrize("N,K", [(384, 512), (256, 4096), (1000, 1024)])
def test_grouped_gemm_matches_oracle(M, N, K):
    w = synthetic.make_w(N, K, 14)
    codes_w, sw_dev = ops.quant_w_int4(w.to(DEV))
    pw = ops.pack_w_int4(codes_w, sw_dev)
    qw, sw = O.quant_w_int4(w)
    r, c = synthetic.make_scales(N, K, 14)
    a = 1.0 / c
    x = synthetic.make_x(M, K, 14 + M)
    codes, sxg = ops.quant_act_int4_grouped(x.to(DEV), a.to(DEV), True, True)
    y = ops.gemm_w4a4_int4_grouped(codes, sxg, pw, r.to(DEV))
    _lib.device_status(0)
    qx, s = O.quant_act_int4_grouped(x, a, 128, True, True)
    assert torch.equal(codes.cpu(), qx)
    acc = O.acc_int32(qx, qw)
    ref = O.epilogue_grouped(acc, sw, r, s)
    ref64 = O.epilogue_grouped(acc, sw, r, s, torch.float64)
    got = y.cpu()
    assert ((got.double() - ref64).abs().max() / ref64.abs().max()).item() < 1e-5
    assert ((got - ref).abs().max() / ref.abs().max()).item() < 1e-5
    # finer scales -> closer to the unquantised product than the per-token variant
    yb = ops.gemm_w4a4_int4_grouped(codes, sxg, pw, r.to(DEV), out_dtype=torch.bfloat16)
    assert torch.equal(yb, y.to(torch.bfloat16))


def test_grouped_scales_reduce_the_quantisation_error():
    M, N, K = 32, 512, 4096
    w = synthetic.make_w(N, K, 15)
    codes_w, sw_dev = ops.quant_w_int4(w.to(DEV))
    pw = ops.pack_w_int4(codes_w, sw_dev)
    x = synthetic.make_x(M, K, 15)  # 1 % outlier channels x 20
    exact = x.double() @ O.dequant_w(*O.quant_w_int4(w), dtype=torch.float64).T
    c1, s1 = ops.quant_act_int4(x.to(DEV), None, None, False)
    y_tok = ops.gemm_w4a4_int4(c1, s1, pw, None).double().cpu()
    cg, sg = ops.quant_act_int4_grouped(x.to(DEV), None, False, False)
    y_grp = ops.gemm_w4a4_int4_grouped(cg, sg, pw, None).double().cpu()
    err_tok = (y_tok - exact).pow(2).sum()
    err_grp = (y_grp - exact).pow(2).sum()
    assert err_grp < 0.5 * err_tok
