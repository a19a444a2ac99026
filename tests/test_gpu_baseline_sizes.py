"""Parity at the full sizes of the benchmark configurations.  The GPU runs the whole problem; the
CPU oracle checks a seeded sample of token rows and output columns (rows of a GEMM are
independent, so a sample of rows x columns is checked exactly as a whole matrix would be):
activation codes / scales and weight codes bit-exact, fp32 outputs < 1e-5 of the fp32 oracle
epilogue (the benchmark tolerance is 1e-3), FP4 outputs < 1e-3 of the fp64 de-quantised matmul."""
import pytest
import torch

from dualquant_b200 import _lib, ops, synthetic
from oracle import dq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _sample(n, count, seed):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randperm(n, generator=g)[: min(n, count)].sort().values
    # always include the edges of the matrix and of a 128-row tile
    extra = torch.tensor([0, min(n - 1, 127), min(n - 1, 128), n - 1])
    return torch.unique(torch.cat([idx, extra]))


_WEIGHTS = {}


def _int4_weight(N, K, seed):
    """(bf16 weight on CPU, packed artefact on the GPU, device codes) - cached per shape."""
    key = (N, K, seed)
    if key not in _WEIGHTS:
        _WEIGHTS.clear()  # one large weight at a time
        w = synthetic.make_w(N, K, seed)
        codes, sw = ops.quant_w_int4(w.to(DEV))
        _WEIGHTS[key] = (w, ops.pack_w_int4(codes, sw), codes, sw)
    return _WEIGHTS[key]


# ---- config 1: every linear of a Llama-3.1-8B layer at every M of the decode sweep --------------
@pytest.mark.parametrize("name,K,N", synthetic.LLAMA31_8B_LINEARS)
@pytest.mark.parametrize("M", synthetic.DECODE_M)
def test_config1_decode_sweep_shapes(name, K, N, M):
    w, pw, codes_w, sw_dev = _int4_weight(N, K, 21)
    r, c = synthetic.make_scales(N, K, 21)
    a = 1.0 / c
    x = synthetic.make_x(M, K, 100 + M)
    y = ops.linear_w4a4_int4(x.to(DEV), a.to(DEV), None, pw, r.to(DEV), scale_fp16=True)
    _lib.device_status(0)
    cols = _sample(N, 192, M)
    qw, sw = O.quant_w_int4(w[cols])
    assert torch.equal(codes_w[cols.to(DEV)].cpu(), qw)
    assert torch.equal(sw_dev[cols.to(DEV)].cpu().view(torch.int16), sw.view(torch.int16))
    qx, sx, _ = O.quant_act_int4(x, a, None, True)
    ref = O.epilogue(O.acc_int32(qx, qw), sw, r[cols], sx)
    got = y[:, cols.to(DEV)].cpu()
    assert ((got.double() - ref.double()).abs().max() / ref.double().abs().max()).item() < 1e-5
    ref64 = O.dequant_matmul(qx, sx, qw, sw, r[cols])
    assert ((got.double() - ref64).abs().max() / ref64.abs().max()).item() < 1e-5


def test_config1_accumulators_bit_exact_on_real_shapes():
    """Per-group int32 sums on the widest (gate+up) and the deepest (down) linear, M = 128."""
    for name, K, N in (("gate_up", 4096, 28672), ("down", 14336, 4096)):
        w, pw, _, _ = _int4_weight(N, K, 21)
        x = synthetic.make_x(128, K, 7)
        qx, _, _ = O.quant_act_int4(x, None, None, True)
        acc = ops.gemm_w4a4_int4_acc(qx.to(DEV), pw)
        rows = _sample(128, 16, 1)
        cols = _sample(N, 48, 2)
        qw, _ = O.quant_w_int4(w[cols])
        ref = O.acc_int32(qx[rows], qw)
        got = acc[rows.to(DEV)][:, cols.to(DEV)].cpu()
        assert torch.equal(got, ref.to(torch.int32))
        _lib.device_status(0)


# ---- config 2: prefill MLP, M = 8192, R4 online Hadamard of size 14336 in front of down_proj ----
def test_config2_prefill_mlp_full_size():
    M, H, I = 8192, 4096, 14336
    rows = _sample(M, 96, 3)
    # gate+up linear, bf16 output
    w_gu, pw_gu, _, _ = _int4_weight(2 * I, H, 31)
    r_gu, c_gu = synthetic.make_scales(2 * I, H, 31)
    a_gu = 1.0 / c_gu
    x = synthetic.make_x(M, H, 31)
    gu = ops.linear_w4a4_int4(x.to(DEV), a_gu.to(DEV), None, pw_gu, r_gu.to(DEV),
                              out_dtype=torch.bfloat16, scale_fp16=True)
    _lib.device_status(0)
    cols = _sample(2 * I, 160, 4)
    qx, sx, _ = O.quant_act_int4(x[rows], a_gu, None, True)
    qw, sw = O.quant_w_int4(w_gu[cols])
    ref = O.epilogue(O.acc_int32(qx, qw), sw, r_gu[cols], sx)
    got = gu[rows.to(DEV)][:, cols.to(DEV)].float().cpu()
    assert ((got - ref).abs() <= 2.0 ** -8 * ref.abs() + 1e-30).all()  # one bf16 rounding of the fp32 result
    # SiLU(gate) * up in bf16 + R4 (28 x 512) + per-token quantiser, fused; then the down GEMM
    r_dn, c_dn = synthetic.make_scales(H, I, 32)
    a_dn = 1.0 / c_dn
    hk, kk = O.get_hadK(I)
    had_dev = ops.Hadamard(_lib.HAD_FULL, kk, 0, O.full_hadamard_scale(I), hk.to(DEV))
    codes, sxd = ops.quant_act_int4_gated(gu[:, :I], gu[:, I:], a_dn.to(DEV), had_dev, True)
    gu_rows = gu[rows.to(DEV)].cpu()
    h = torch.nn.functional.silu(gu_rows[:, :I]) * gu_rows[:, I:]
    qh, sh, _ = O.quant_act_int4(h, a_dn, ("full", hk, kk), True)
    diff = (codes[rows.to(DEV)].cpu().int() - qh.int()).abs()
    # expf differs in the last ulp between CPU and GPU: a handful of bf16 roundings may move a code
    assert diff.max() <= 1 and (diff > 0).float().mean() < 2e-3
    assert torch.allclose(sxd[rows.to(DEV)].cpu(), sh, rtol=2e-3)
    del pw_gu
    w_dn, pw_dn, _, _ = _int4_weight(H, I, 33)
    y = ops.gemm_w4a4_int4(codes, sxd, pw_dn, r_dn.to(DEV))
    _lib.device_status(0)
    cols_d = _sample(H, 160, 5)
    qw_d, sw_d = O.quant_w_int4(w_dn[cols_d])
    # the GEMM itself against the oracle on the GPU's own codes (bit-exact integers, fp32 epilogue)
    ref_d = O.epilogue(O.acc_int32(codes[rows.to(DEV)].cpu(), qw_d), sw_d, r_dn[cols_d], sxd[rows.to(DEV)].cpu())
    got_d = y[rows.to(DEV)][:, cols_d.to(DEV)].cpu()
    assert ((got_d.double() - ref_d.double()).abs().max() / ref_d.double().abs().max()).item() < 1e-5
    # the same projection on the FP8 tensor-core path (the quantiser writes E4M3 code bytes, the
    # weight's byte form is derived from the artefact): the whole [8192, 4096] output bit for bit
    x8, sx8 = ops.quant_act_int4_gated(gu[:, :I], gu[:, I:], a_dn.to(DEV), had_dev, True, e4m3=True)
    assert torch.equal(sx8, sxd)
    y8 = ops.gemm_w4a4_int4_e4m3(x8, sx8, pw_dn.bytes_e4m3(), pw_dn, r_dn.to(DEV))
    _lib.device_status(0)
    assert torch.equal(y8, y)
    del x8, y8
    # and the plain (ungated) Hadamard quantiser at this size, bit-exact
    hb = h.to(torch.bfloat16)
    c2, s2 = ops.quant_act_int4(hb.to(DEV), a_dn.to(DEV), had_dev, True)
    q2, sx2, _ = O.quant_act_int4(hb, a_dn, ("full", hk, kk), True)
    assert torch.equal(c2.cpu(), q2) and torch.equal(s2.cpu(), sx2)


# ---- config 3: block-scaled FP4 on the Qwen2.5-7B shapes, M = 4096 ----------------------------------
@pytest.mark.parametrize("fmt_name", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("name,K,N", synthetic.QWEN25_7B_LINEARS)
def test_config3_fp4_prefill_shapes(fmt_name, name, K, N):
    fmt = _lib.FP4_MXFP4 if fmt_name == "mxfp4" else _lib.FP4_NVFP4
    M = 4096
    w = synthetic.make_w(N, K, 41)
    pw = ops.pack_w_fp4(w.to(DEV), fmt)
    r, c = synthetic.make_scales(N, K, 41)
    a = 1.0 / c
    x = synthetic.make_x(M, K, 41)
    y = ops.linear_w4a4_fp4(x.to(DEV), a.to(DEV), pw, r.to(DEV))
    _lib.device_status(0)
    rows, cols = _sample(M, 64, 6), _sample(N, 128, 7)
    x32 = x[rows].float() * a
    if fmt_name == "mxfp4":
        xd = O.quant_mxfp4(x32)[2]
        wd = O.quant_mxfp4(w[cols].float())[2]
    else:
        xd = O.quant_nvfp4(x32)[3]
        ts = float((w.float().abs().max() / 2688.0).item())
        wd = O.quant_nvfp4(w[cols].float(), ts)[3]
    ref = (xd.double() @ wd.double().T) * r[cols].double()
    got = y[rows.to(DEV)][:, cols.to(DEV)].double().cpu()
    assert ((got - ref).abs().max() / ref.abs().max()).item() < 1e-3


@pytest.mark.parametrize("fmt_name", ["mxfp4", "nvfp4"])
def test_config3_fp4_decode_shapes(fmt_name):
    fmt = _lib.FP4_MXFP4 if fmt_name == "mxfp4" else _lib.FP4_NVFP4
    M = 16
    for name, K, N in synthetic.QWEN25_7B_LINEARS:
        w = synthetic.make_w(N, K, 43)
        pw = ops.pack_w_fp4(w.to(DEV), fmt)
        r, c = synthetic.make_scales(N, K, 43)
        a = 1.0 / c
        x = synthetic.make_x(M, K, 43)
        y = ops.linear_w4a4_fp4(x.to(DEV), a.to(DEV), pw, r.to(DEV))
        _lib.device_status(0)
        cols = _sample(N, 128, 8)
        x32 = x.float() * a
        if fmt_name == "mxfp4":
            xd, wd = O.quant_mxfp4(x32)[2], O.quant_mxfp4(w[cols].float())[2]
        else:
            xd = O.quant_nvfp4(x32)[3]
            wd = O.quant_nvfp4(w[cols].float(), float((w.float().abs().max() / 2688.0).item()))[3]
        ref = (xd.double() @ wd.double().T) * r[cols].double()
        got = y[:, cols.to(DEV)].double().cpu()
        assert ((got - ref).abs().max() / ref.abs().max()).item() < 1e-3
