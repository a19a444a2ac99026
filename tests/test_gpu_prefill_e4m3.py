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


# ------------------------------------------------------------------------------------------
# the exchange kernels of the token-sharded prompt pass, one rank at a time on one GPU: every
# "peer" buffer is a local array, and no kernel waits for another
# ------------------------------------------------------------------------------------------
def _exchange_ctx(world, rank, tq, hidden, part, codes, sx, flags):
    ctx = _lib.ExchangeCtx()
    ctx.world, ctx.rank = world, rank
    for p in range(world):
        ctx.part_ptrs[p] = part[p].data_ptr()
        ctx.codes_ptrs[p] = codes[p].data_ptr()
        ctx.sx_ptrs[p] = sx[p].data_ptr()
        ctx.flag_ptrs[p] = flags[p].data_ptr()
    ctx.tokens_per_rank, ctx.hidden = tq, hidden
    return ctx


@pytest.mark.parametrize("world,tq,N,K", [(1, 512, 256, 512), (2, 256, 128, 1024), (4, 256, 384, 256), (8, 512, 256, 128)])
def test_scatter_gemm_puts_every_tile_into_its_owners_slot(world, tq, N, K):
    """dq_gemm_w4a4_int4_e4m3_scatter as each rank in turn: slot `rank` of owner p's partial buffer
    must hold rows [p * tq, (p + 1) * tq) of the plain GEMM's bf16 output, and nothing else moves."""
    import ctypes

    M = world * tq
    codes_w, sw, pw = _weights(N, K, 11)
    r, _ = synthetic.make_scales(N, K, 11)
    x8, sx = ops.quant_act_int4(synthetic.make_x(M, K, 13).to(DEV), None, None, False, e4m3=True)
    want = ops.gemm_w4a4_int4_e4m3(x8, sx, pw.bytes_e4m3(), pw, r.to(DEV), out_dtype=torch.bfloat16)
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for rank in range(world):
        part = torch.full((world, world, tq, N), 7.0, dtype=torch.bfloat16, device=DEV)
        codes = torch.zeros(world, M, N, dtype=torch.uint8, device=DEV)
        sxg = torch.zeros(world, M, dtype=torch.float32, device=DEV)
        flags = torch.zeros(world, 8, dtype=torch.int32, device=DEV)
        ctx = _exchange_ctx(world, rank, tq, N, part, codes, sxg, flags)
        rc = lib.dq_gemm_w4a4_int4_e4m3_scatter(ctypes.c_void_p(x8.data_ptr()), ctypes.c_void_p(sx.data_ptr()),
                                                ctypes.c_void_p(pw.bytes_e4m3().data_ptr()),
                                                ctypes.c_void_p(pw.sw_t.data_ptr()), ctypes.c_void_p(r.to(DEV).data_ptr()),
                                                M, N, K, 128, ctypes.byref(ctx), stream)
        assert rc == 0, _lib.last_error()
        _lib.device_status(0)
        for p in range(world):
            assert torch.equal(part[p, rank], want[p * tq:(p + 1) * tq]), (rank, p)
            others = [s for s in range(world) if s != rank]
            assert bool((part[p, others] == 7.0).all())


def test_scatter_gemm_rejects_shapes_it_cannot_tile():
    import ctypes

    codes_w, sw, pw = _weights(128, 128, 1)
    x8, sx = ops.quant_act_int4(synthetic.make_x(300, 128, 1).to(DEV), None, None, False, e4m3=True)
    part = torch.zeros(1, 1, 300, 128, dtype=torch.bfloat16, device=DEV)
    dummy = torch.zeros(1, 300 * 128, dtype=torch.uint8, device=DEV)
    ctx = _exchange_ctx(1, 0, 300, 128, part, dummy, torch.zeros(1, 300, device=DEV),
                        torch.zeros(1, 8, dtype=torch.int32, device=DEV))
    rc = _lib.load().dq_gemm_w4a4_int4_e4m3_scatter(
        ctypes.c_void_p(x8.data_ptr()), ctypes.c_void_p(sx.data_ptr()), ctypes.c_void_p(pw.bytes_e4m3().data_ptr()),
        ctypes.c_void_p(pw.sw_t.data_ptr()), None, 300, 128, 128, 128, ctypes.byref(ctx),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and "tokens_per_rank" in _lib.last_error()


@pytest.mark.parametrize("world", [1, 2, 8])
def test_exchange_sum_and_push(world):
    """Owner side: x += bf16(rank-ordered fp32 sum of the partial slots); then the owner's codes and
    token scales land in its slice of every rank's gathered buffers."""
    import ctypes

    tq, H = 256, 128
    g = torch.Generator(device=DEV).manual_seed(world)
    part = torch.randn(world, world, tq, H, generator=g, device=DEV).to(torch.bfloat16)
    codes = torch.zeros(world, world * tq, H, dtype=torch.uint8, device=DEV)
    sxg = torch.zeros(world, world * tq, dtype=torch.float32, device=DEV)
    flags = torch.zeros(world, 8, dtype=torch.int32, device=DEV)
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rank = world - 1
    ctx = _exchange_ctx(world, rank, tq, H, part, codes, sxg, flags)
    x = torch.randn(tq, H, generator=g, device=DEV).to(torch.bfloat16)
    acc = part[rank, 0].float()
    for p in range(1, world):
        acc = acc + part[rank, p].float()
    want = (x.float() + acc.to(torch.bfloat16).float()).to(torch.bfloat16)
    assert lib.dq_exchange_sum(ctypes.byref(ctx), ctypes.c_void_p(x.data_ptr()), stream) == 0
    assert torch.equal(x, want)
    mine = torch.randint(0, 256, (tq, H), generator=g, device=DEV, dtype=torch.uint8)
    smine = torch.rand(tq, generator=g, device=DEV)
    assert lib.dq_exchange_push(ctypes.byref(ctx), ctypes.c_void_p(mine.data_ptr()), ctypes.c_void_p(smine.data_ptr()),
                                stream) == 0
    for p in range(world):
        assert torch.equal(codes[p, rank * tq:(rank + 1) * tq], mine)
        assert torch.equal(sxg[p, rank * tq:(rank + 1) * tq], smine)
        assert int(codes[p].sum().item()) == int(mine.sum().item())  # nothing outside the slice
    _lib.device_status(0)
