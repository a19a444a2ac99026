"""GPU parity tests of the int4 path: every call goes through the C ABI (ctypes) and is compared
with the CPU oracle on the same seeded inputs.  Integer work is bit-exact; fp32 outputs within
1e-3 relative (tolerance from the benchmark specification)."""
import numpy as np
import pytest
import torch

from dualquant_b200 import _lib, ops, synthetic
from oracle import dq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL_TOL = 1e-3


def _rel_err(y, ref):
    return ((y.double() - ref.double()).abs().max() / ref.double().abs().max()).item()


def _status_ok():
    _lib.device_status(0)


def _operands(M, N, K, seed=0, scale_fp16=True):
    x = synthetic.make_x(M, K, seed)
    w = synthetic.make_w(N, K, seed)
    r, c = synthetic.make_scales(N, K, seed)
    a = 1.0 / c
    qx, sx, _ = O.quant_act_int4(x, a, None, scale_fp16)
    qw, sw = O.quant_w_int4(w)
    return x, w, r, a, qx, sx, qw, sw


# ------------------------------------------------------------------------------------------
# weights
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("N,K", [(128, 128), (200, 384), (4096, 4096)])
def test_quant_and_pack_weights_bit_exact(N, K):
    w = synthetic.make_w(N, K, 5)
    w[3, :128] = 0  # an all-zero group
    qw, sw = O.quant_w_int4(w)
    codes, sw_g = ops.quant_w_int4(w.to(DEV))
    assert torch.equal(codes.cpu(), qw)
    assert torch.equal(sw_g.cpu().view(torch.int16), sw.view(torch.int16))
    pw = ops.pack_w_int4(codes, sw_g)
    assert torch.equal(pw.w_packed.cpu(), O.stream_pack_int4(qw, sw))
    assert torch.equal(pw.sw_t.cpu(), O.stream_pack_scales(sw))
    assert torch.equal(ops.unpack_w_int4(pw).cpu(), qw)
    # the reference's packed form as the source gives the same artefact
    pw2 = ops.pack_w_int4(None, sw_g, ref_packed=O.ref_pack_int4(qw).to(DEV))
    assert torch.equal(pw2.w_packed, pw.w_packed)
    _status_ok()


def test_pack_from_reference_golden(golden):
    packed = torch.from_numpy(golden["refpack_packed"])
    codes = O.ref_unpack_int4(packed)
    sw = torch.ones(32, 2, dtype=torch.float16)
    pw = ops.pack_w_int4(None, sw.to(DEV), ref_packed=packed.to(DEV))
    assert torch.equal(ops.unpack_w_int4(pw).cpu(), codes)


# ------------------------------------------------------------------------------------------
# activation quantiser
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,K", [(1, 128), (3, 4096), (17, 14336), (5, 18944), (64, 8), (2, 40000)])
@pytest.mark.parametrize("scale_fp16", [False, True])
def test_act_quant_bit_exact(M, K, scale_fp16):
    x = synthetic.make_x(M, K, 3)
    if M > 1:
        x[1] = 0  # all-zero token -> scale 1, codes 0
    _, c = synthetic.make_scales(8, K, 3)
    a = 1.0 / c
    qx, sx, _ = O.quant_act_int4(x, a, None, scale_fp16)
    codes, sxg = ops.quant_act_int4(x.to(DEV), a.to(DEV), None, scale_fp16)
    assert torch.equal(sxg.cpu(), sx)
    assert torch.equal(codes.cpu(), qx)
    # without a column scale
    qx0, sx0, _ = O.quant_act_int4(x, None, None, scale_fp16)
    codes0, sx0g = ops.quant_act_int4(x.to(DEV), None, None, scale_fp16)
    assert torch.equal(codes0.cpu(), qx0) and torch.equal(sx0g.cpu(), sx0)
    _status_ok()


def test_act_quant_empty_and_strided():
    x = synthetic.make_x(6, 512, 1).to(DEV)
    codes, sx = ops.quant_act_int4(x[:0], None, None, False)
    assert codes.shape == (0, 512) and sx.shape == (0,)
    wide = torch.zeros(6, 1024, dtype=torch.bfloat16, device=DEV)
    wide[:, :512] = x
    c1, s1 = ops.quant_act_int4(wide[:, :512], None, None, False)  # ldx = 1024
    c2, s2 = ops.quant_act_int4(x, None, None, False)
    assert torch.equal(c1, c2) and torch.equal(s1, s2)


def test_act_quant_golden_reference_cast(golden):
    x32 = torch.from_numpy(golden["cast_in"])
    out = ops.fakequant_act_int4(x32.to(DEV), None, None, False)
    assert torch.equal(out.cpu(), torch.from_numpy(golden["cast_out"]))


def test_act_quant_rejects_bad_arguments():
    x = synthetic.make_x(2, 100, 1).to(DEV)  # K % 8 != 0
    with pytest.raises(ValueError):
        ops.quant_act_int4(x, None, None, False)
    with pytest.raises(RuntimeError):
        ops.quant_act_int4(synthetic.make_x(2, 128, 1), None, None, False)  # CPU tensor


# ------------------------------------------------------------------------------------------
# Hadamard
# ------------------------------------------------------------------------------------------
def _full_had(K):
    had, k = O.get_hadK(K)
    return ops.Hadamard(_lib.HAD_FULL, k, 0, O.full_hadamard_scale(K),
                        None if had is None else had.to(DEV)), ("full", had, k)


# (up to 64 rows with a factor order divisible by four and segments of 128 ... 1024 take the
# four-CTA cluster kernel: 14336 = 28 x 512, 28672 = 28 x 1024, 7168 = 28 x 256, 3584 = 28 x 128;
# 65 rows: the one-CTA kernel again)
@pytest.mark.parametrize("M,K", [(3, 896), (2, 14336), (4, 1024), (2, 64), (3, 4096), (1, 2048), (2, 28 * 1024),
                                 (2, 32768), (2, 7168), (64, 3584), (65, 3584)])
def test_full_hadamard_bit_exact(M, K):
    hd, ohad = _full_had(K)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(M, K, generator=g)
    ref = O.hadamard_full(x, ohad[1], ohad[2])
    got = ops.hadamard_f32(x.to(DEV), hd)
    assert torch.equal(got.cpu(), ref)
    xb = synthetic.make_x(M, K, 4)
    qx, sx, _ = O.quant_act_int4(xb, None, ohad, True)
    codes, sxg = ops.quant_act_int4(xb.to(DEV), None, hd, True)
    assert torch.equal(codes.cpu(), qx) and torch.equal(sxg.cpu(), sx)
    _status_ok()


# Row lengths of a row-parallel down_proj shard (14336 / 8, / 4, / 2) and other short segments: several
# threads share a column pair of the matrix stage.  70 rows: one 512-thread CTA per row; 500 rows: three
# 256-thread CTAs per SM.  1536 = 12 x 128 and 2560 = 40 x 64 -> 20 x 128 go through the generic order.
@pytest.mark.parametrize("M,K", [(70, 1792), (500, 1792), (500, 3584), (70, 7168), (500, 7168), (70, 14336),
                                 (500, 14336), (500, 896), (500, 1536), (70, 2560)])
def test_full_hadamard_many_rows_bit_exact(M, K):
    hd, ohad = _full_had(K)
    xb = synthetic.make_x(M, K, 11)
    _, c = synthetic.make_scales(8, K, 11)
    a = 1.0 / c
    qx, sx, _ = O.quant_act_int4(xb, a, ohad, False)
    codes, sxg = ops.quant_act_int4(xb.to(DEV), a.to(DEV), hd, False)
    assert torch.equal(codes.cpu(), qx) and torch.equal(sxg.cpu(), sx)
    x32 = xb.float()
    got = ops.hadamard_f32(x32.to(DEV), hd)
    assert torch.equal(got.cpu(), O.hadamard_full(x32, ohad[1], ohad[2]))
    _status_ok()


@pytest.mark.parametrize("K,d", [(4096, 128), (256, 8), (1024, 64), (8192, 128)])
def test_partial_hadamard_bit_exact(K, d):
    M = 5
    hd = ops.Hadamard(_lib.HAD_PARTIAL, 1, d, O.partial_hadamard_scale(K // d), None)
    xb = synthetic.make_x(M, K, 6)
    _, c = synthetic.make_scales(8, K, 6)
    a = 1.0 / c
    qx, sx, _ = O.quant_act_int4(xb, a, ("partial", d), False)
    codes, sxg = ops.quant_act_int4(xb.to(DEV), a.to(DEV), hd, False)
    assert torch.equal(codes.cpu(), qx) and torch.equal(sxg.cpu(), sx)


# 64 rows and more of 2 ... 32 heads x 128 take the register-only kernel (16 or 32 lanes per row);
# 63 rows and head sizes other than 128 stay on the one-CTA-per-row kernel.
@pytest.mark.parametrize("M,K,d", [(64, 4096, 128), (333, 4096, 128), (300, 2048, 128), (301, 1024, 128),
                                   (65, 512, 128), (1000, 256, 128), (63, 4096, 128), (300, 1024, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_partial_hadamard_many_rows_bit_exact(M, K, d, dtype):
    hd = ops.Hadamard(_lib.HAD_PARTIAL, 1, d, O.partial_hadamard_scale(K // d), None)
    xb = synthetic.make_x(M, K, 12)
    _, c = synthetic.make_scales(8, K, 12)
    a = 1.0 / c
    for fp16 in (False, True):
        qx, sx, _ = O.quant_act_int4(xb, a, ("partial", d), fp16)
        codes, sxg = ops.quant_act_int4(xb.to(DEV).to(dtype), a.to(DEV), hd, fp16)
        assert torch.equal(codes.cpu(), qx) and torch.equal(sxg.cpu(), sx)
    x8, sx8 = ops.quant_act_int4(xb.to(DEV).to(dtype), a.to(DEV), hd, True, e4m3=True)
    assert torch.equal(x8, ops.codes_to_e4m3(codes)) and torch.equal(sx8, sxg)
    _status_ok()


@pytest.mark.parametrize("K", [1536, 2560, 1152, 1664, 3840, 6912, 4480, 4992, 11008])
def test_full_hadamard_other_orders_bit_exact(K):
    """Every order of the reference's table (12, 40, 36, 52, 60, 108, 140, 156, 172) times a power of
    two: transform and codes against the oracle, whose matrices are the reference's own."""
    from dualquant_b200 import quarot

    had, k = O.get_hadK(K)
    hk, kk = quarot.get_hadK(K)
    assert kk == k and torch.equal(hk, had)
    hd = ops.Hadamard(_lib.HAD_FULL, k, 0, quarot.full_hadamard_scale(K), hk.to(DEV))
    g = torch.Generator().manual_seed(K)
    x = torch.randn(3, K, generator=g)
    ref = O.hadamard_full(x, had, k)
    got = ops.hadamard_f32(x.to(DEV), hd)
    assert torch.equal(got.cpu(), ref)
    xb = synthetic.make_x(3, K, 6)
    _, c = synthetic.make_scales(8, K, 6)
    a = 1.0 / c
    qx, sx, _ = O.quant_act_int4(xb, a, ("full", had, k), False)
    codes, sxg = ops.quant_act_int4(xb.to(DEV), a.to(DEV), hd, False)
    assert torch.equal(codes.cpu(), qx) and torch.equal(sxg.cpu(), sx)
    _status_ok()


def test_hadamard_golden(golden):
    x = torch.from_numpy(golden["hadfull_in"])
    hd, _ = _full_had(896)
    got = ops.hadamard_f32(x.to(DEV), hd).cpu()
    ref = torch.from_numpy(golden["hadfull_out"])
    assert torch.allclose(got, ref, rtol=0, atol=2e-6 * ref.abs().max().item())


# ------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------
def _gpu_weight(qw, sw):
    return ops.pack_w_int4(qw.to(DEV), sw.to(DEV))


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (3, 128, 256), (16, 256, 512), (17, 384, 384),
                                   (100, 200, 640), (130, 128, 1024)])
def test_gemm_accumulators_bit_exact(M, N, K):
    _, _, _, _, qx, sx, qw, sw = _operands(M, N, K, seed=M)
    pw = _gpu_weight(qw, sw)
    acc = ops.gemm_w4a4_int4_acc(qx.to(DEV), pw)
    _status_ok()
    assert torch.equal(acc.cpu(), O.acc_int32(qx, qw))


def test_gemm_accumulators_extreme_codes():
    # every product at its largest magnitude: (-8) * (-8) * 128 = 8192 per group
    M, N, K = 16, 128, 256
    qx = torch.full((M, K), -8, dtype=torch.int8)
    qw = torch.full((N, K), -8, dtype=torch.int8)
    qw[::2] = 7
    pw = _gpu_weight(qw, torch.ones(N, K // 128, dtype=torch.float16))
    acc = ops.gemm_w4a4_int4_acc(qx.to(DEV), pw)
    assert torch.equal(acc.cpu(), O.acc_int32(qx, qw))


@pytest.mark.parametrize("M,N,K,tn,split", [
    (1, 128, 128, 0, 0), (1, 256, 1024, 16, 1), (1, 256, 1024, 16, 8), (8, 384, 512, 16, 4),
    (16, 4096, 4096, 0, 0), (20, 256, 512, 32, 2), (32, 512, 1024, 32, 8), (50, 200, 640, 64, 1),
    (64, 256, 2048, 64, 4), (128, 256, 512, 128, 1), (128, 384, 1024, 128, 2),
    (300, 640, 384, 128, 1), (7, 136, 256, 0, 0), (7, 136, 256, 16, 1),
    # both tcgen05 kernels at every tile: 1000 + tile = int8 weight tiles in shared memory,
    # 2000 + tile = weights through tensor memory
    (9, 256, 640, 1016, 1), (20, 256, 512, 1032, 2), (64, 256, 2048, 1064, 4), (50, 200, 640, 1064, 1),
    (130, 384, 1024, 2128, 1), (128, 256, 512, 2128, 2), (300, 640, 384, 2128, 1), (40, 136, 384, 2064, 1),
    (33, 256, 384, 2064, 1), (128, 128, 128, 2128, 1),
    # decode-batch (register-path) kernel: negative token_tile = token capacity
    (1, 256, 1024, -8, 1), (1, 256, 1024, -8, 8), (8, 384, 512, -8, 4), (5, 200, 384, -8, 2),
    (16, 4096, 4096, -16, 0), (12, 256, 512, -16, 2), (16, 128, 14336, -16, 8),
    (20, 256, 512, -32, 2), (32, 512, 1024, -32, 8), (3, 136, 256, -32, 1),
])
def test_gemm_output_matches_oracle(M, N, K, tn, split):
    _, _, r, _, qx, sx, qw, sw = _operands(M, N, K, seed=M + N)
    pw = _gpu_weight(qw, sw)
    y = ops.gemm_w4a4_int4(qx.to(DEV), sx.to(DEV), pw, r.to(DEV), token_tile=tn, split_k=split)
    _status_ok()
    ref64 = O.dequant_matmul(qx, sx, qw, sw, r)
    assert _rel_err(y.cpu(), ref64) < REL_TOL
    ref32 = O.epilogue(O.acc_int32(qx, qw), sw, r, sx)
    assert _rel_err(y.cpu(), ref32) < 1e-5
    # bf16 output and no row scale
    yb = ops.gemm_w4a4_int4(qx.to(DEV), sx.to(DEV), pw, None, out_dtype=torch.bfloat16,
                            token_tile=tn, split_k=split)
    refb = O.dequant_matmul(qx, sx, qw, sw, None)
    assert _rel_err(yb.float().cpu(), refb) < 8e-3  # bf16 rounding of the output


def test_gemm_is_deterministic_and_linear_in_scales():
    M, N, K = 16, 512, 4096
    _, _, r, _, qx, sx, qw, sw = _operands(M, N, K, seed=9)
    pw = _gpu_weight(qw, sw)
    args = (qx.to(DEV), sx.to(DEV), pw, r.to(DEV))
    y1 = ops.gemm_w4a4_int4(*args)
    y2 = ops.gemm_w4a4_int4(*args)
    assert torch.equal(y1, y2)
    y3 = ops.gemm_w4a4_int4(qx.to(DEV), (2 * sx).to(DEV), pw, (4 * r).to(DEV))
    assert torch.equal(y3, 8 * y1)  # power-of-two scaling is exact in fp32


def test_config0_full_size_against_oracle():
    # M=2048, K=4096, N=4096, seed 0: the reference's own CPU-runnable configuration
    M, N, K = 2048, 4096, 4096
    x, w, r, a, qx, sx, qw, sw = _operands(M, N, K, seed=0)
    codes, sxg = ops.quant_act_int4(x.to(DEV), a.to(DEV), None, True)
    assert torch.equal(codes.cpu(), qx) and torch.equal(sxg.cpu(), sx)
    cw, swg = ops.quant_w_int4(w.to(DEV))
    assert torch.equal(cw.cpu(), qw)
    pw = ops.pack_w_int4(cw, swg)
    y = ops.gemm_w4a4_int4(codes, sxg, pw, r.to(DEV))
    _status_ok()
    ref = O.dequant_matmul(qx, sx, qw, sw, r, dtype=torch.float32)
    assert _rel_err(y.cpu(), ref) < REL_TOL
    # one-call linear gives the same bits as the two-step path
    y2 = ops.linear_w4a4_int4(x.to(DEV), a.to(DEV), None, pw, r.to(DEV), scale_fp16=True)
    assert torch.equal(y2, y)


def test_gemm_rejects_bad_arguments():
    qx = torch.zeros(4, 192, dtype=torch.int8, device=DEV)
    pw = ops.PackedInt4Weight(torch.zeros(2 * 8448, dtype=torch.uint8, device=DEV),
                              torch.ones(128, dtype=torch.float16, device=DEV), 128, 192)
    with pytest.raises(ValueError):
        ops.gemm_w4a4_int4(qx, torch.ones(4, device=DEV), pw)  # K % 128 != 0


def test_act_quant_rounding_boundaries_and_tiny_scales():
    # rows built so that x / s lands exactly on and next to half-integers, plus rows whose scale
    # is denormal-small (1/s overflows): the fast rounding path must still equal IEEE division
    K = 1024
    g = torch.Generator().manual_seed(5)
    rows = []
    base = torch.zeros(K)
    base[0] = 7.0  # absmax 7 -> s = 1 exactly: elements are their own quotients
    halves = (torch.arange(K - 1) % 15 - 7).float() + 0.5
    r1 = base.clone(); r1[1:] = halves
    r2 = base.clone(); r2[1:] = torch.nextafter(halves, torch.full_like(halves, 10.0))
    r3 = base.clone(); r3[1:] = torch.nextafter(halves, torch.full_like(halves, -10.0))
    rows += [r1, r2, r3]
    rows.append(torch.randn(K, generator=g) * 1e-41)   # denormal magnitudes
    rows.append(torch.randn(K, generator=g) * 3e-39)
    rows.append(torch.randn(K, generator=g) * 1e30)
    x = torch.stack(rows)
    for scale_fp16 in (False, True):
        q, s, _ = O.quant_act_int4(x, None, None, scale_fp16)
        ref = q.float() * s.reshape(-1, 1)
        got = ops.fakequant_act_int4(x.to(DEV), None, None, scale_fp16).cpu()
        assert torch.equal(got, ref)


def test_gated_quantiser_matches_bf16_silu_mul():
    # SiLU(gate) * up in bf16 fused in front of the Hadamard quantiser; expf differs in the last
    # ulp between CPU and GPU, so a handful of bf16 roundings (hence codes) may differ
    M, K = 6, 14336
    g = torch.Generator().manual_seed(11)
    gu = (torch.randn(M, 2 * K, generator=g) * 1.5).to(torch.bfloat16)
    gate, up = gu[:, :K], gu[:, K:]
    h = torch.nn.functional.silu(gate) * up
    _, c = synthetic.make_scales(8, K, 11)
    a = 1.0 / c
    hd, ohad = _full_had(K)
    gud = gu.to(DEV)
    for had_dev, had_cpu in ((None, None), (hd, ohad)):
        qx, sx, _ = O.quant_act_int4(h, a, had_cpu, True)
        codes, sxg = ops.quant_act_int4_gated(gud[:, :K], gud[:, K:], a.to(DEV), had_dev, True)
        diff = (codes.cpu().int() - qx.int()).abs()
        assert diff.max() <= 1 and (diff > 0).float().mean() < 2e-3
        assert torch.allclose(sxg.cpu(), sx, rtol=2e-3)


# ------------------------------------------------------------------------------------------
# RMSNorm fused into the quantiser
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,K,with_w", [(1, 4096, False), (8, 4096, True), (33, 1024, True),
                                        (5, 14336, False), (130, 256, True)])
def test_quant_act_rmsnorm_matches_norm_then_quant(M, K, with_w):
    g = torch.Generator().manual_seed(M * 7 + K)
    x = (torch.randn(M, K, generator=g) * 3.0).bfloat16()
    x[:, : max(1, K // 100)] *= 20  # outlier channels
    w = (1.0 + 0.1 * torch.randn(K, generator=g)).bfloat16() if with_w else None
    a = torch.exp(torch.randn(K, generator=g) * 0.3)
    codes, sx = ops.quant_act_int4_rmsnorm(x.to(DEV), None if w is None else w.to(DEV), 1e-5, a.to(DEV))
    _status_ok()
    normed = O.rmsnorm_bf16(x, w, 1e-5)
    qref, sref, _ = O.quant_act_int4(normed, a, scale_fp16=False)
    # the sum of squares is reduced in another order and rsqrt may differ in its last bit:
    # a normalised value can land on the other side of a bf16 or code rounding boundary
    diff = (codes.cpu().int() - qref.int()).abs()
    assert int(diff.max()) <= 1
    assert float((diff != 0).float().mean()) < 2e-3
    assert torch.allclose(sx.cpu(), sref, rtol=8e-3, atol=0)


def test_quant_act_rmsnorm_rejects_bad_arguments():
    x = torch.randn(4, 256, device=DEV).bfloat16()
    with pytest.raises(ValueError):
        ops.quant_act_int4_rmsnorm(x.float(), None, 1e-5)
    with pytest.raises(ValueError):
        ops.quant_act_int4_rmsnorm(x, torch.ones(128, device=DEV).bfloat16(), 1e-5)
    with pytest.raises(ValueError):
        ops.quant_act_int4_rmsnorm(x, None, -1.0)


# ------------------------------------------------------------------------------------------
# every GEMM kernel forms the same fp32 sums in the same order
# ------------------------------------------------------------------------------------------
def test_all_gemm_kernels_bit_identical_on_random_shapes():
    """Decode kernel, tensor-memory-operand and shared-memory-operand tcgen05 kernels at every
    token tile: without split-K each adds float(acc_g) * sw_g in group order, so their outputs
    must be equal bit for bit (a cheap detector for races in the pipelines)."""
    import random
    rnd = random.Random(0)
    g = torch.Generator(device=DEV).manual_seed(1)
    for _ in range(60):
        M = rnd.choice([1, 7, 8, 9, 16, 17, 32, 33, 64, 100, 128, 129, 300, 513])
        N = rnd.choice([128, 136, 256, 640, 1024, 4096])
        K = 128 * rnd.choice([1, 2, 3, 5, 8, 13, 32, 56])
        codes = torch.randint(-8, 8, (M, K), generator=g, device=DEV, dtype=torch.int8)
        sx = torch.rand(M, generator=g, device=DEV) + 0.5
        wq = torch.randint(-8, 8, (N, K), generator=g, device=DEV, dtype=torch.int8)
        sw = (torch.rand(N, K // 128, generator=g, device=DEV) * 0.02 + 0.001).half()
        r = torch.rand(N, generator=g, device=DEV) + 0.5
        pw = ops.pack_w_int4(wq, sw)
        tiles = [t for t in (-8, -16, -32) if M <= -t]
        for tn in (16, 32, 64, 128):
            if tn == 16 and M > 64:
                continue
            tiles += [1000 + tn, 2000 + tn]
        outs = [ops.gemm_w4a4_int4(codes, sx, pw, r, token_tile=t, split_k=1) for t in tiles]
        for t, y in zip(tiles[1:], outs[1:]):
            assert torch.equal(y, outs[0]), (M, N, K, tiles[0], t)
        auto1 = ops.gemm_w4a4_int4(codes, sx, pw, r)
        auto2 = ops.gemm_w4a4_int4(codes, sx, pw, r)
        assert torch.equal(auto1, auto2), (M, N, K)
        # the persistent FP8-path kernel (codes as E4M3 bytes, fp32 group sums): same bits again
        y8 = ops.gemm_w4a4_int4_e4m3(ops.codes_to_e4m3(codes), sx, ops.expand_w_e4m3(pw), pw, r)
        assert torch.equal(y8, outs[0]), (M, N, K, "e4m3")
    _status_ok()


@pytest.mark.parametrize("M,K", [(1024, 2048), (1100, 4096), (1024, 14336)])
def test_quant_act_many_rows_bit_exact(M, K):
    """Row counts at which the quantiser switches to its many-rows launch shape."""
    x = synthetic.make_x(M, K, K)
    a = torch.exp(torch.randn(K, generator=torch.Generator().manual_seed(K)) * 0.3)
    codes, sx = ops.quant_act_int4(x.to(DEV), a.to(DEV), None, True)
    _status_ok()
    q, s, _ = O.quant_act_int4(x, a, None, scale_fp16=True)
    assert torch.equal(codes.cpu(), q)
    assert torch.equal(sx.cpu(), s)
