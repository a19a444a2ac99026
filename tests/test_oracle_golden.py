"""The CPU oracle against vectors produced by the reference's own code
(tests/golden/make_golden.py).  Integer / bit-pattern work is compared exactly."""
import numpy as np
import torch

from oracle import dq_oracle as O


def _bf16(arr):
    return torch.from_numpy(arr.copy()).view(torch.bfloat16)


def test_had28_is_paley2(golden):
    had = O.paley2_hadamard(13)
    assert torch.equal(had, torch.from_numpy(golden["had28"]).float())
    assert torch.equal(had @ had.T, 28 * torch.eye(28))
    h, k = O.get_hadK(14336)
    assert k == 28 and torch.equal(h, had)
    assert O.get_hadK(32) == (None, 1)


def test_act_cast_matches_rtn_cast(golden):
    x32 = torch.from_numpy(golden["cast_in"])
    q, s, _ = O.quant_act_int4(x32, None, None, scale_fp16=False)
    deq = q.float() * s.reshape(-1, 1)
    assert torch.equal(deq, torch.from_numpy(golden["cast_out"]))
    assert s[5].item() == 1.0 and int(q[5].abs().max()) == 0  # all-zero token
    assert int(q.max()) <= 7 and int(q.min()) >= -8


def test_weight_cast_group128(golden):
    # the reference keeps the group scale in fp32; with the scale forced back to fp32 the oracle's
    # codes must reproduce the reference's fake-quant weight exactly
    w = torch.from_numpy(golden["wcast_in"])
    N, K = w.shape
    wg = w.reshape(N, K // 128, 128)
    amax = wg.abs().amax(-1, keepdim=True)
    s = amax / 7
    s[amax == 0] = 1
    q = (wg / s).round().clamp(-8, 7)
    assert torch.equal((q * s).reshape(N, K), torch.from_numpy(golden["wcast_out"]))
    # the oracle's fp16-scale variant stays within half a step of the input
    codes, sw = O.quant_w_int4(w.to(torch.bfloat16))
    deq = O.dequant_w(codes, sw)
    step = sw.float().repeat_interleave(128, dim=1)
    assert torch.all((deq - w).abs() <= 0.5 * step * (1 + 2e-3) + 1e-12)


def _perm_case(golden, tag, had):
    x = _bf16(golden[f"perm_{tag}_x"])
    a = torch.from_numpy(golden[f"perm_{tag}_a"])
    q, s, _ = O.quant_act_int4(x, a, had, scale_fp16=False)
    xq = (q.float() * s.reshape(-1, 1)).to(torch.bfloat16)
    ref = _bf16(golden[f"perm_{tag}_xq_bf16"])
    return xq, ref, q, s


def test_perm_linear_plain_bit_exact(golden):
    xq, ref, q, s = _perm_case(golden, "plain", None)
    # value equality: the reference keeps the sign of a rounded-to-zero element (-0.0), int8
    # codes do not; every non-zero element must match bit for bit
    assert torch.equal(xq.float(), ref.float())
    w = _bf16(golden["perm_plain_w_bf16"])
    y = torch.nn.functional.linear(xq, w)
    assert torch.equal(y.float(), _bf16(golden["perm_plain_y_bf16"]).float())


def test_perm_linear_partial_hadamard_bit_exact(golden):
    xq, ref, _, _ = _perm_case(golden, "partial", ("partial", 8))
    assert torch.equal(xq.float(), ref.float())


def test_perm_linear_full_hadamard(golden):
    # the 28x28 stage of the reference is an fp32 matmul with unspecified summation order:
    # allow codes to differ at rounding ties, but only rarely and only by one step
    had, k = O.get_hadK(896)
    xq, ref, q, s = _perm_case(golden, "full", ("full", had, k))
    diff = (xq.float() - ref.float()).abs()
    step = s.reshape(-1, 1)
    flips = (diff > 1e-3 * step).float().mean().item()
    assert flips < 2e-3
    assert torch.all(diff <= step * 1.01)


def test_hadamard_full_fp32(golden):
    x = torch.from_numpy(golden["hadfull_in"])
    had, k = O.get_hadK(896)
    got = O.hadamard_full(x, had, k)
    ref = torch.from_numpy(golden["hadfull_out"])
    assert torch.allclose(got, ref, rtol=0, atol=2e-6 * ref.abs().max().item())
    # orthogonality: applying it twice with the transpose structure returns the input norm
    assert torch.allclose(got.norm(dim=1), x.norm(dim=1), rtol=1e-5)


def test_reference_packing_round_trip(golden):
    packed = torch.from_numpy(golden["refpack_packed"])
    codes = O.ref_unpack_int4(packed)
    assert torch.equal(O.ref_pack_int4(codes), packed)
    scale = _bf16(golden["refpack_scale_bf16"]).float()
    deq = codes.float().reshape(32, 2, 128) * scale.reshape(32, 2, 1)
    assert torch.equal(deq.reshape(32, 256), torch.from_numpy(golden["refpack_dequant"]))
    # streaming layout: pure permutation of the same nibbles (tile 0, group 0, row 0, chunk 0)
    sp = O.stream_pack_int4(codes, torch.ones(32, 2, dtype=torch.float16))
    assert sp.numel() == 2 * 8448  # 32 rows padded to one 128-row tile, two k groups
    first = sp[:16].to(torch.int16)
    lo = first & 0xF
    lo = torch.where(lo > 7, lo - 16, lo)
    hi = first >> 4
    hi = torch.where(hi > 7, hi - 16, hi)
    assert torch.equal(lo, codes[0, 0:16].to(torch.int16))
    assert torch.equal(hi, codes[0, 16:32].to(torch.int16))
    # the tile ends with its 128 fp16 scales (1.0 for real rows, 0 for padding rows)
    tail = sp[8192:8448].view(torch.float16)
    assert torch.equal(tail[:32], torch.ones(32, dtype=torch.float16)) and tail[32:].abs().max() == 0
    # second k group of row 0 starts one tile later
    nxt = sp[8448:8448 + 16].to(torch.int16) & 0xF
    nxt = torch.where(nxt > 7, nxt - 16, nxt)
    assert torch.equal(nxt, codes[0, 128:144].to(torch.int16))


def test_float_to_fp4(golden):
    x = torch.from_numpy(golden["fp4_in"])
    assert torch.equal(O.float_to_fp4(x), torch.from_numpy(golden["fp4_out"]))


def test_acc_and_epilogue_agree_with_dequant_matmul():
    g = torch.Generator().manual_seed(3)
    M, N, K = 9, 40, 384
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    r = torch.exp(torch.randn(N, generator=g) * 0.3).half().float()
    qx, sx, _ = O.quant_act_int4(x, None, None, True)
    qw, sw = O.quant_w_int4(w)
    acc = O.acc_int32(qx, qw)
    ref_acc = torch.einsum("mgk,ngk->mng", qx.long().reshape(M, 3, 128), qw.long().reshape(N, 3, 128))
    assert torch.equal(acc.long(), ref_acc)
    y32 = O.epilogue(acc, sw, r, sx)
    y64 = O.dequant_matmul(qx, sx, qw, sw, r)
    assert torch.allclose(y32.double(), y64, rtol=1e-5, atol=1e-6 * y64.abs().max().item())


def test_mxfp4_block_cast_matches_convert_to_mxfp(golden):
    # legacy_vendor/torch_quant.py:359-375 run on CPU by the fixture generator, block 32
    x = torch.from_numpy(golden["mxfp4_in"])
    _, e8m0, deq = O.quant_mxfp4(x, 32)
    assert torch.equal(deq, torch.from_numpy(golden["mxfp4_out"]))
    assert int(e8m0.reshape(16, -1)[3, 2]) == 0  # the all-zero block carries the smallest exponent


def test_nvfp4_block_scale_rounding_matches_quantize_scale_e4m3(golden):
    # scale_formats.py:39-45: clamp to [2^-6, 448], cast to E4M3 (round to nearest even) and back.
    # Feed each grid value as "amax / 6 / ts" of a block of 16 and read the block scale back.
    want = torch.from_numpy(golden["e4m3_scale_in"])
    x = torch.zeros(want.numel(), 16)
    x[:, 0] = want * 6.0
    exact = (x[:, 0] / 6.0) == want  # keep only grid points that survive the *6 /6 round trip
    _, bs, _, _ = O.quant_nvfp4(x, tensor_scale=1.0)
    ref = torch.from_numpy(golden["e4m3_scale_out"])
    assert int(exact.sum()) > 500
    assert torch.equal(bs.reshape(-1)[exact], ref[exact])
    assert float(bs.min()) == 2.0 ** -6  # zero / tiny blocks are clamped to the smallest normal


def test_bf16_arithmetic_branch_matches_reference(golden):
    # PermLinear without activation scale / Hadamard quantises the bf16 tensor in bf16 arithmetic
    x = _bf16(golden["perm_noscale_x"])
    q, s, deq = O.quant_act_int4_bf16_arith(x)
    assert torch.equal(deq, _bf16(golden["perm_noscale_xq_bf16"]))
    assert s[3].item() == 1.0 and int(q[3].abs().max()) == 0
    # and it is not the fp32 quantiser: some codes differ
    q32, _, _ = O.quant_act_int4(x, None, None, False)
    assert not torch.equal(q32, q)
