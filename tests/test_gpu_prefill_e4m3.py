"""The int4 GEMM on the FP8 tensor-core path (prefill): E4M3 byte operands, fp32 group sums.

Integer work, so everything here is bit-exact: the byte forms against a table of the sixteen codes,
the GEMM against the oracle's integer accumulation and epilogue and against the int8-path kernel."""
import pytest
import torch

from dualquant_b200 import _lib, decoder, ops, quarot, synthetic
from oracle import dq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# E4M3 bytes of the integers a two's-complement nibble stands for: 0..7, then -8..-1
E4M3_OF_NIBBLE = torch.tensor([0x00, 0x38, 0x40, 0x44, 0x48, 0x4A, 0x4C, 0x4E,
                               0xD0, 0xCE, 0xCC, 0xCA, 0xC8, 0xC4, 0xC0, 0xB8], dtype=torch.uint8)


def _as_e4m3(codes: torch.Tensor) -> torch.Tensor:
    return E4M3_OF_NIBBLE.to(codes.device)[codes.long() & 15]


def _weights(N, K, seed):
    codes_w, sw = ops.quant_w_int4(synthetic.make_w(N, K, seed).to(DEV))
    return codes_w, sw, ops.pack_w_int4(codes_w, sw)


def test_the_table_is_e4m3():
    vals = torch.tensor(list(range(8)) + list(range(-8, 0)), dtype=torch.float32)
    assert torch.equal(E4M3_OF_NIBBLE.view(torch.float8_e4m3fn).float(), vals)


@pytest.mark.parametrize("N,K", [(128, 128), (200, 1024), (384, 4096)])
def test_weight_bytes_are_the_codes(N, K):
    codes_w, _, pw = _weights(N, K, 3)
    w8 = ops.expand_w_e4m3(pw)
    assert w8.shape == (N, K) and torch.equal(w8, _as_e4m3(codes_w))
    assert torch.equal(ops.codes_to_e4m3(codes_w), w8)
    _lib.device_status(0)


@pytest.mark.parametrize("M,K", [(5, 512), (300, 4096), (64, 14336)])
def test_quantisers_write_e4m3_codes_on_request(M, K):
    """Every quantiser front end (plain, fp32 rows, online Hadamard, RMSNorm, gated) with the flag:
    same scales, and code bytes that are the int8 codes' E4M3 form."""
    x = synthetic.make_x(M, K, 4).to(DEV)
    x[1] = 0  # an all-zero token
    up = synthetic.make_x(M, K, 5).to(DEV)
    a = (1.0 / synthetic.make_scales(8, K, 5)[1]).to(DEV)
    hk, kk = quarot.get_hadK(K)
    had = ops.Hadamard(_lib.HAD_FULL, kk, 0, quarot.full_hadamard_scale(K), None if hk is None else hk.to(DEV))
    for fn in (lambda e: ops.quant_act_int4(x, a, None, True, e4m3=e),
               lambda e: ops.quant_act_int4(x, None, None, False, bf16_arith=True, e4m3=e),
               lambda e: ops.quant_act_int4(x.float(), a, None, False, e4m3=e),
               lambda e: ops.quant_act_int4(x, a, had, False, e4m3=e),
               lambda e: ops.quant_act_int4_rmsnorm(x, torch.ones(K, dtype=torch.bfloat16, device=DEV), 1e-5, a, e4m3=e),
               lambda e: ops.quant_act_int4_gated(x, up, a, had, e4m3=e)):
        codes, sx = fn(False)
        bytes_, sx8 = fn(True)
        assert bytes_.dtype == torch.uint8 and torch.equal(sx, sx8)
        assert torch.equal(bytes_, _as_e4m3(codes))
    _lib.device_status(0)


# ragged token and row counts (tiles are 256 tokens x 128 rows), one group and many, N not a multiple
# of 8 (direct stores instead of the bulk store)
@pytest.mark.parametrize("M,N,K", [(256, 128, 128), (1, 128, 256), (300, 200, 1024), (777, 1001, 2048),
                                   (1024, 384, 4096), (513, 256, 14336)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_equals_oracle_and_int8_path(M, N, K, dtype):
    codes_w, sw, pw = _weights(N, K, 5)
    r, c = synthetic.make_scales(N, K, 5)
    x = synthetic.make_x(M, K, 6).to(DEV)
    codes, sx = ops.quant_act_int4(x, (1.0 / c).to(DEV), None, True)
    x8, sx8 = ops.quant_act_int4(x, (1.0 / c).to(DEV), None, True, e4m3=True)
    got = ops.gemm_w4a4_int4_e4m3(x8, sx8, ops.expand_w_e4m3(pw), pw, r.to(DEV), out_dtype=dtype)
    _lib.device_status(0)
    want = ops.gemm_w4a4_int4(codes, sx, pw, r.to(DEV), out_dtype=dtype)
    assert torch.equal(got, want)
    if M * N * K <= 300 * 200 * 1024:
        ref = O.epilogue(O.acc_int32(codes.cpu(), codes_w.cpu()), sw.cpu(), r, sx.cpu()).to(dtype)
        assert torch.equal(got.cpu(), ref)


@pytest.mark.parametrize("M,N,K", [(512, 256, 1024), (300, 1001, 512)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_with_residual(M, N, K, dtype):
    codes_w, sw, pw = _weights(N, K, 7)
    r, _ = synthetic.make_scales(N, K, 7)
    x8, sx = ops.quant_act_int4(synthetic.make_x(M, K, 8).to(DEV), None, None, False, e4m3=True)
    w8 = pw.bytes_e4m3()
    res = torch.randn(M, N, generator=torch.Generator().manual_seed(1)).to(dtype).to(DEV)
    plain = ops.gemm_w4a4_int4_e4m3(x8, sx, w8, pw, r.to(DEV), out_dtype=dtype)
    fused = ops.gemm_w4a4_int4_e4m3(x8, sx, w8, pw, r.to(DEV), residual=res)
    assert torch.equal(fused, plain + res)
    buf = res.clone()  # in place: the residual is also the output
    ops.gemm_w4a4_int4_e4m3(x8, sx, w8, pw, r.to(DEV), out=buf, residual=buf)
    _lib.device_status(0)
    assert torch.equal(buf, fused)


def test_many_tiles_per_cta_and_token_blocks():
    """More tiles than SMs, several token blocks (K = 14336 puts 11 token tiles in a block): every
    tile is computed once and lands in its place."""
    M, N, K = 16 * 256, 1280, 14336
    codes_w, sw, pw = _weights(N, K, 9)
    x = synthetic.make_x(M, K, 10).to(DEV)
    codes, sx = ops.quant_act_int4(x, None, None, False)
    want = ops.gemm_w4a4_int4(codes, sx, pw, None, out_dtype=torch.bfloat16)
    got = ops.gemm_w4a4_int4_e4m3(ops.codes_to_e4m3(codes), sx, pw.bytes_e4m3(), pw, None, out_dtype=torch.bfloat16)
    _lib.device_status(0)
    assert torch.equal(got, want)


def test_linear_entry_takes_the_fp8_path_with_the_larger_scratch():
    M, N, K = 1024, 512, 2048
    _, _, pw = _weights(N, K, 11)
    r, c = synthetic.make_scales(N, K, 11)
    x = synthetic.make_x(M, K, 12).to(DEV)
    small = ops.linear_scratch_bytes(M, N, K, prefill=False)
    large = ops.linear_scratch_bytes(M, N, K)
    assert large >= small + N * K
    assert ops.linear_scratch_bytes(M - 1, N, K) == ops.linear_scratch_bytes(M - 1, N, K, prefill=False)
    outs = []
    for nbytes in (small, large):
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        outs.append(ops.linear_w4a4_int4(x, (1.0 / c).to(DEV), None, pw, r.to(DEV), out_dtype=torch.bfloat16,
                                         scale_fp16=True, scratch=scratch))
    _lib.device_status(0)
    assert torch.equal(outs[0], outs[1])


def test_decoder_linear_rows_do_not_depend_on_the_batch_they_arrive_in():
    """Per-token quantisation makes every output row a function of its input row alone, so a batch
    above the prefill threshold (FP8 path) must reproduce the rows of two batches below it."""
    gen = torch.Generator(device=DEV).manual_seed(3)
    N, K = 384, 1024
    lin = decoder.W4A4Linear(N, K, torch.device(DEV), gen, None)
    M = 2 * (lin.PREFILL_TOKENS - 128)
    assert M >= lin.PREFILL_TOKENS
    x = synthetic.make_x(M, K, 13).to(DEV)
    ln = torch.ones(K, dtype=torch.bfloat16, device=DEV)
    res = torch.randn(M, N, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV)
    h = M // 2
    for whole, parts in ((lin(x), (lin(x[:h]), lin(x[h:]))),
                         (lin(x, residual=res), (lin(x[:h], residual=res[:h].contiguous()),
                                                 lin(x[h:], residual=res[h:].contiguous()))),
                         (lin.normed(x, ln, 1e-5), (lin.normed(x[:h], ln, 1e-5), lin.normed(x[h:], ln, 1e-5))),
                         (lin.gated(x, x.flip(0).contiguous()),
                          (lin.gated(x[:h], x.flip(0)[:h].contiguous()), lin.gated(x[h:], x.flip(0)[h:].contiguous())))):
        assert torch.equal(whole, torch.cat(parts))
    _lib.device_status(0)
