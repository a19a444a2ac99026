"""Size-independent properties of the CPU oracle (no GPU): what must hold for any input."""
import torch
from hypothesis import given, settings, strategies as st

from oracle import dq_oracle as O


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 9), st.sampled_from([128, 256, 640]), st.integers(0, 2 ** 31 - 1), st.booleans())
def test_act_quantiser_properties(M, K, seed, fp16_scale):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, K, generator=g) * 3).bfloat16()
    a = torch.exp(torch.randn(K, generator=g) * 0.3)
    q, s, x32 = O.quant_act_int4(x, a, None, scale_fp16=fp16_scale)
    assert q.dtype == torch.int8 and int(q.min()) >= -8 and int(q.max()) <= 7
    assert torch.all(s > 0)
    # the dequantised value is within half a step (plus the fp16 rounding of the scale)
    deq = q.float() * s.reshape(-1, 1)
    slack = 1e-3 if fp16_scale else 1e-6
    inside = (x32 / s.reshape(-1, 1)).abs() <= 7.5  # an fp16-rounded scale may clip the largest element
    assert torch.all(((deq - x32).abs() <= (0.5 + slack) * s.reshape(-1, 1) + 1e-12) | ~inside)
    # idempotence: quantising the de-quantised tensor (scale 1 column vector) gives the same codes
    q2, s2, _ = O.quant_act_int4(deq, None, None, scale_fp16=False)
    assert torch.equal(q2.float() * s2.reshape(-1, 1), deq)


@settings(max_examples=15, deadline=None)
@given(st.integers(1, 5), st.integers(1, 3), st.integers(1, 4), st.integers(0, 2 ** 31 - 1))
def test_gemm_oracle_linearity_and_packing(M, tiles, groups, seed):
    g = torch.Generator().manual_seed(seed)
    N, K = tiles * 128 - 7, groups * 128
    qx = torch.randint(-8, 8, (M, K), generator=g, dtype=torch.int8)
    qw = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int8)
    sw = (torch.rand(N, groups, generator=g) * 0.02 + 1e-3).half()
    sx = torch.rand(M, generator=g) + 0.5
    r = torch.rand(N, generator=g) + 0.5
    acc = O.acc_int32(qx, qw)
    assert acc.dtype in (torch.int32, torch.int64) and int(acc.abs().max()) <= 8 * 8 * 128
    y = O.epilogue(acc, sw, r, sx)
    # linear in the token scale and in the row scale
    assert torch.allclose(O.epilogue(acc, sw, r, 2 * sx), 2 * y, rtol=1e-6, atol=0)
    assert torch.allclose(O.epilogue(acc, sw, 3 * r, sx), 3 * y, rtol=1e-6, atol=0)
    # the reference packing round-trips and the streaming layout has the advertised size
    packed = O.ref_pack_int4(qw)
    assert torch.equal(O.ref_unpack_int4(packed), qw)
    stream = O.stream_pack_int4(qw, sw)
    assert stream.numel() == tiles * groups * 8448
    # every code of the matrix appears once: the nibble histogram of the code bytes matches
    body = stream.reshape(tiles, groups, 8448)[:, :, :8192].reshape(-1)
    nibbles = torch.cat([body & 0xF, body >> 4]).long()
    hist = torch.bincount(nibbles, minlength=16)
    want = torch.bincount((qw.long() & 0xF).reshape(-1), minlength=16)
    want[0] += (tiles * 128 - N) * K  # zero rows that pad the last tile
    assert torch.equal(hist, want)


@settings(max_examples=15, deadline=None)
@given(st.integers(1, 4), st.sampled_from([32, 64, 256]), st.integers(0, 2 ** 31 - 1))
def test_fp4_quantisers_stay_on_the_grid(M, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * 5
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    q, e, deq = O.quant_mxfp4(x)
    assert torch.isin(q.abs(), grid).all()
    assert torch.all((deq - x).abs() <= x.abs().reshape(M, K // 32, 32).amax(-1, keepdim=True)
                     .repeat_interleave(32, -1).reshape(M, K) * 0.26 + 1e-12)
    q2, bs, ts, deq2 = O.quant_nvfp4(x, None)
    assert torch.isin(q2.abs(), grid).all() and torch.all(ts > 0)
