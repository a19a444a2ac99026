"""Block-scaled FP4 quantisers (MXFP4 / NVFP4) through the C ABI against the oracle: packed
E2M1 codes, scale bytes and second-level scales bit-exact, de-quantised values equal."""
import pytest
import torch

from dualquant_b200 import _lib, formats, ops, synthetic
from oracle import dq_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _x(M, K, seed):
    x = synthetic.make_x(M, K, seed)
    if M > 2:
        x[1] = 0  # all-zero row
        x[2, :64] = 0  # all-zero blocks
    return x


@pytest.mark.parametrize("M,K", [(1, 32), (3, 128), (5, 3584), (2, 18944), (4, 4096)])
@pytest.mark.parametrize("use_a", [False, True])
def test_mxfp4_bit_exact(M, K, use_a):
    x = _x(M, K, 7)
    a = None
    x32 = x.float()
    if use_a:
        _, c = synthetic.make_scales(8, K, 7)
        a = 1.0 / c
        x32 = x32 * a
    q, e8, deq = O.quant_mxfp4(x32)
    codes, sf, rs = ops.quant_fp4(x.to(DEV), _lib.FP4_MXFP4, None if a is None else a.to(DEV))
    assert rs is None
    assert torch.equal(sf.cpu(), e8)
    assert torch.equal(codes.cpu(), O.pack_fp4(q))
    fq = ops.fakequant_fp4(x.to(DEV), _lib.FP4_MXFP4, None if a is None else a.to(DEV))
    assert torch.equal(fq.cpu(), deq)
    _lib.device_status(0)


@pytest.mark.parametrize("fmt", [_lib.FP4_MXFP4, _lib.FP4_NVFP4])
@pytest.mark.parametrize("M,K", [(520, 3584), (512, 18944), (600, 2048), (513, 8192)])
def test_fp4_quant_many_rows_bit_exact(fmt, M, K):
    """Hundreds of rows, every launch shape of the quantiser (1-4 vectors per thread) against the oracle."""
    x = _x(M, K, 11)
    _, c = synthetic.make_scales(8, K, 11)
    a = 1.0 / c
    x32 = x.float() * a
    codes, sf, rs = ops.quant_fp4(x.to(DEV), fmt, a.to(DEV))
    if fmt == _lib.FP4_MXFP4:
        q, e8, deq = O.quant_mxfp4(x32)
        assert torch.equal(sf.cpu(), e8)
    else:
        q, bs, ts, deq = O.quant_nvfp4(x32, None)
        assert torch.equal(sf.cpu(), O.e4m3_byte(bs))
        assert torch.equal(rs.cpu(), ts)
    assert torch.equal(codes.cpu(), O.pack_fp4(q))
    fq = ops.fakequant_fp4(x.to(DEV), fmt, a.to(DEV))
    assert torch.equal(fq.cpu(), deq)
    # scale bytes written straight in the order the GEMM streams = the re-ordered row-major bytes
    codes2, sfa, rs2 = ops.quant_fp4(x.to(DEV), fmt, a.to(DEV), None, atoms=True)
    assert torch.equal(codes2, codes)
    assert torch.equal(sfa.reshape(-1), ops.fp4_sf_to_atoms(sf, K, fmt).reshape(-1))
    _lib.device_status(0)


@pytest.mark.parametrize("M,K", [(1, 16), (3, 128), (5, 3584), (2, 18944), (4, 4096)])
@pytest.mark.parametrize("per_tensor", [False, True])
def test_nvfp4_bit_exact(M, K, per_tensor):
    x = _x(M, K, 9)
    x32 = x.float()
    ts_dev = None
    ts_val = None
    if per_tensor:
        ts_dev = ops.nvfp4_tensor_scale(x.to(DEV))
        ts_val = float(ts_dev.item())
        ref_ts = x32.abs().max() / 2688.0
        assert ts_val == float(ref_ts)
    q, bs, ts, deq = O.quant_nvfp4(x32, ts_val)
    codes, sf, rs = ops.quant_fp4(x.to(DEV), _lib.FP4_NVFP4, None, ts_dev)
    assert torch.equal(sf.cpu(), O.e4m3_byte(bs))
    assert torch.equal(codes.cpu(), O.pack_fp4(q))
    if not per_tensor:
        assert torch.equal(rs.cpu(), ts)
    fq = ops.fakequant_fp4(x.to(DEV), _lib.FP4_NVFP4, None, ts_dev)
    assert torch.equal(fq.cpu(), deq)
    _lib.device_status(0)


def test_mxfp4_cast_matches_reference_convert_to_mxfp(golden):
    """The library's MXFP4 cast against the output of the reference's own convert_to_mxfp
    (legacy_vendor/torch_quant.py:359-375, block 32) recorded in the golden fixtures: zero block,
    tiny and huge magnitudes, block maxima on the grid, elements on rounding ties."""
    x = torch.from_numpy(golden["mxfp4_in"])
    want = torch.from_numpy(golden["mxfp4_out"])
    fq = ops.fakequant_fp4(x.to(DEV), _lib.FP4_MXFP4)
    assert torch.equal(fq.cpu(), want)
    assert torch.equal(formats.make_format("mxfp4").cast(x.to(DEV)).cpu(), want)
    _lib.device_status(0)


def test_nvfp4_block_scale_matches_reference_e4m3_quantiser(golden):
    """NVFP4 block-scale bytes against the reference's quantize_scale_e4m3 (scale_formats.py:39-45:
    clamp to [2^-6, 448], E4M3 round-to-nearest-even) on a grid of scale values."""
    want = torch.from_numpy(golden["e4m3_scale_in"])
    x = torch.zeros(want.numel(), 16)
    x[:, 0] = want * 6.0
    exact = (x[:, 0] / 6.0) == want
    one = torch.ones(1, device=DEV)
    _, sf, _ = ops.quant_fp4(x.to(DEV), _lib.FP4_NVFP4, None, one)
    got = sf.cpu().view(torch.float8_e4m3fn).float().reshape(-1)
    ref = torch.from_numpy(golden["e4m3_scale_out"])
    assert torch.equal(got[exact], ref[exact])
    _lib.device_status(0)


def test_element_rounding_matches_reference_table(golden):
    # blocks whose exponent is 0 (absmax in [4, 8)): the MXFP4 element is float_to_fp4(x) itself
    grid = torch.from_numpy(golden["fp4_in"])
    want = torch.from_numpy(golden["fp4_out"])
    keep = grid.abs() <= 6.0
    vals, ref = grid[keep], want[keep]
    n = (vals.numel() // 31) * 31
    rows = vals[:n].reshape(-1, 31)
    x = torch.cat([rows, torch.full((rows.shape[0], 1), 6.0)], dim=1)  # pin the block exponent to 0
    fq = ops.fakequant_fp4(x.to(DEV), _lib.FP4_MXFP4).cpu()
    assert torch.equal(fq[:, :31].reshape(-1), ref[:n])
    f = formats.make_format("mxfp4")
    assert torch.equal(f.cast_element_only(grid), want)


def test_format_specs():
    f = formats.make_format("nvfp4")
    assert (f.name, f.block_size, f.max_val) == ("nvfp4", 16, 6.0)
    with pytest.raises(ValueError):
        formats.make_format("nvfp4", block_size=32)
    w = synthetic.make_w(64, 256, 1).to(DEV)
    got = f.cast(w)
    ts = float((w.float().abs().max() / 2688.0).item())
    _, _, _, deq = O.quant_nvfp4(w.float().cpu(), ts)
    assert got.dtype == w.dtype and torch.equal(got.float().cpu(), deq.to(torch.bfloat16).float())
    fm = formats.make_format("mxfp4", block_size=32)
    _, _, deq2 = O.quant_mxfp4(w.float().cpu())
    assert torch.equal(fm.cast(w.float()).cpu(), deq2)


# ------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------
def _fp4_reference(x, a, w, r, fmt):
    x32 = x.float() * a if a is not None else x.float()
    if fmt == _lib.FP4_MXFP4:
        _, _, xd = O.quant_mxfp4(x32)
        _, _, wd = O.quant_mxfp4(w.float())
    else:
        _, _, _, xd = O.quant_nvfp4(x32)
        ts = float((w.float().abs().max() / 2688.0).item())
        _, _, _, wd = O.quant_nvfp4(w.float(), ts)
    y = xd.double() @ wd.double().T
    return y * r.double().reshape(1, -1) if r is not None else y


def test_sf_atom_order():
    rows, K = 200, 512
    sf = torch.arange(rows * (K // 16), dtype=torch.int64).remainder(251).to(torch.uint8).reshape(rows, K // 16)
    out = ops.fp4_sf_to_atoms(sf.to(DEV), K, _lib.FP4_NVFP4).cpu()
    nsf = K // 16
    assert out.numel() == 256 * nsf
    for row, k in ((0, 0), (5, 3), (37, 4), (131, 17), (199, 31)):
        tile, rr = divmod(row, 128)
        atom = tile * (nsf // 4) + k // 4
        idx = atom * 512 + (rr % 32) * 16 + (rr // 32) * 4 + k % 4
        assert out[idx] == sf[row, k]
    assert out[(1 * (nsf // 4)) * 512 + (8 % 32) * 16 + 3 * 4] == 0  # row 128+104 = 232 is padding


@pytest.mark.parametrize("fmt", [_lib.FP4_MXFP4, _lib.FP4_NVFP4])
@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (16, 256, 512), (130, 200, 768), (1, 128, 3584),
                                   (16, 384, 2048), (40, 136, 1024), (16, 3584, 18944)])
def test_fp4_gemm_matches_dequant_matmul(fmt, M, N, K):
    x = synthetic.make_x(M, K, M + 1)
    w = synthetic.make_w(N, K, N + 2)
    r, c = synthetic.make_scales(N, K, 3)
    a = 1.0 / c
    pw = ops.pack_w_fp4(w.to(DEV), fmt)
    y = ops.linear_w4a4_fp4(x.to(DEV), a.to(DEV), pw, r.to(DEV))
    _lib.device_status(0)
    ref = _fp4_reference(x, a, w, r, fmt)
    err = ((y.double().cpu() - ref).abs().max() / ref.abs().max()).item()
    assert err < 1e-3, err


@pytest.mark.parametrize("fmt", [_lib.FP4_MXFP4, _lib.FP4_NVFP4])
@pytest.mark.parametrize("M,N,K", [(256, 128, 256), (130, 200, 768), (257, 384, 512), (384, 136, 768),
                                   (1000, 4096, 1024), (70, 128, 512)])
def test_fp4_gemm_token_tiles_agree(fmt, M, N, K):
    """The 128- and the 256-token tile give the same output bit for bit (same products, same
    K order in one fp32 accumulator), full, ragged and single-block tiles alike, and both match
    the de-quantised fp32 matmul."""
    x = synthetic.make_x(M, K, M + 5)
    w = synthetic.make_w(N, K, N + 6)
    r, c = synthetic.make_scales(N, K, 7)
    a = (1.0 / c).to(DEV)
    pw = ops.pack_w_fp4(w.to(DEV), fmt)
    codes, sf, rs = ops.quant_fp4(x.to(DEV), fmt, a, None)
    sfa = ops.fp4_sf_to_atoms(sf, K, fmt)
    y1 = ops.gemm_w4a4_fp4(codes, sfa, rs, pw, r.to(DEV), token_tile=128)
    y2 = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_w4a4_fp4(codes, sfa, rs, pw, r.to(DEV), out=y2, token_tile=256)
    _lib.device_status(0)
    assert torch.equal(y1, y2)
    ref = _fp4_reference(x, a.cpu(), w, r, fmt)
    err = ((y2.double().cpu() - ref).abs().max() / ref.abs().max()).item()
    assert err < 1e-3, err


# Shapes the library sends to the persistent prefill kernel (at least 512 tokens, 256-token tiles
# that fill whole rounds of one tile per SM): one tile per CTA and several, a last token tile of 216
# tokens (two scale-factor blocks) and one of 100 (a single block), rows past N.
@pytest.mark.parametrize("fmt", [_lib.FP4_MXFP4, _lib.FP4_NVFP4])
# (1024 x 5120 and 1000 x 5104 are 160 tiles on 148 SMs: 37 row tiles go to the persistent kernel,
# the last three to the one-tile kernel with split-K)
@pytest.mark.parametrize("M,N,K,dtype", [(728, 6272, 512, torch.float32), (612, 6260, 768, torch.bfloat16),
                                         (2048, 9472, 256, torch.bfloat16), (1024, 5120, 8192, torch.bfloat16),
                                         (1000, 5104, 8192, torch.float32)])
def test_fp4_persistent_kernel_equals_the_one_tile_kernel(fmt, M, N, K, dtype):
    x = synthetic.make_x(M, K, M + 1)
    w = synthetic.make_w(N, K, N + 2)
    r, c = synthetic.make_scales(N, K, 3)
    a = (1.0 / c).to(DEV)
    pw = ops.pack_w_fp4(w.to(DEV), fmt)
    codes, sf, rs = ops.quant_fp4(x.to(DEV), fmt, a, None)
    sfa = ops.fp4_sf_to_atoms(sf, K, fmt)
    want = ops.gemm_w4a4_fp4(codes, sfa, rs, pw, r.to(DEV), out_dtype=dtype, token_tile=128)
    got = torch.full((M, N), float("nan"), dtype=dtype, device=DEV)
    ops.gemm_w4a4_fp4(codes, sfa, rs, pw, r.to(DEV), out=got)  # library's choice: the persistent kernel
    _lib.device_status(0)
    # (rows finished by a split-K launch sum their fp32 partial sums in another order)
    assert torch.allclose(got.float(), want.float(), rtol=2e-6 if dtype == torch.float32 else 2 ** -7, atol=1e-6)
    if N in (6272, 6260, 9472):
        assert torch.equal(got, want)
    ref = _fp4_reference(x, a.cpu(), w, r, fmt)
    err = ((got.double().cpu() - ref).abs().max() / ref.abs().max()).item()
    assert err < (1e-3 if dtype == torch.float32 else 1e-2), err


@pytest.mark.parametrize("fmt", [_lib.FP4_MXFP4, _lib.FP4_NVFP4])
@pytest.mark.parametrize("M,N,K,dtype", [(130, 130, 768, torch.float32), (257, 204, 512, torch.bfloat16),
                                         (40, 136, 768, torch.bfloat16), (129, 200, 512, torch.bfloat16),
                                         (40, 64, 512, torch.float32), (3, 8, 256, torch.bfloat16)])
def test_fp4_gemm_output_pitches_and_dtypes(fmt, M, N, K, dtype):
    """Outputs whose row pitch is not a multiple of 16 bytes take the direct-store epilogue, the
    others the bulk-store one; fp32 and bf16, ragged M and N."""
    x = synthetic.make_x(M, K, M + 21)
    w = synthetic.make_w(N, K, N + 22)
    r, c = synthetic.make_scales(N, K, 23)
    a = (1.0 / c).to(DEV)
    pw = ops.pack_w_fp4(w.to(DEV), fmt)
    codes, sf, rs = ops.quant_fp4(x.to(DEV), fmt, a, None)
    sfa = ops.fp4_sf_to_atoms(sf, K, fmt)
    y = torch.full((M + 1, N), 7.0, dtype=dtype, device=DEV)  # one guard row behind the output
    ops.gemm_w4a4_fp4(codes, sfa, rs, pw, r.to(DEV), out=y[:M])
    _lib.device_status(0)
    assert torch.all(y[M] == 7.0)
    ref = _fp4_reference(x, a.cpu(), w, r, fmt)
    tol = 1e-3 if dtype == torch.float32 else 8e-3  # bf16 output rounding: 2^-8 relative
    err = ((y[:M].double().cpu() - ref).abs().max() / ref.abs().max()).item()
    assert err < tol, err


def test_fp4_wide_tile_rejects_split_k_shapes():
    M, N, K = 16, 256, 2048  # a decode batch: the 128-token path splits K over a cluster
    x = synthetic.make_x(M, K, 1).to(DEV)
    pw = ops.pack_w_fp4(synthetic.make_w(N, K, 2).to(DEV), _lib.FP4_MXFP4)
    codes, sf, rs = ops.quant_fp4(x, _lib.FP4_MXFP4, None, None)
    sfa = ops.fp4_sf_to_atoms(sf, K, _lib.FP4_MXFP4)
    with pytest.raises((RuntimeError, ValueError)):
        ops.gemm_w4a4_fp4(codes, sfa, rs, pw, None, token_tile=256)
    with pytest.raises((RuntimeError, ValueError)):
        ops.gemm_w4a4_fp4(codes, sfa, rs, pw, None, token_tile=64)


@pytest.mark.parametrize("fmt", [_lib.FP4_MXFP4, _lib.FP4_NVFP4])
@pytest.mark.parametrize("M,N,K", [(1, 128, 256), (16, 256, 2048), (16, 3584, 3584), (32, 200, 768), (7, 384, 1024),
                                   (20, 37888, 512)])
def test_fp4_gemm_decode_tile_matches_dequant_matmul(fmt, M, N, K):
    """The 32-token tile (decode batches of up to 32 tokens, with and without split-K over a
    cluster) against the de-quantised fp32 matmul and against the 128-token tile."""
    x = synthetic.make_x(M, K, M + 9)
    w = synthetic.make_w(N, K, N + 10)
    r, c = synthetic.make_scales(N, K, 11)
    a = (1.0 / c).to(DEV)
    pw = ops.pack_w_fp4(w.to(DEV), fmt)
    codes, sf, rs = ops.quant_fp4(x.to(DEV), fmt, a, None)
    sfa = ops.fp4_sf_to_atoms(sf, K, fmt)
    y = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_w4a4_fp4(codes, sfa, rs, pw, r.to(DEV), out=y, token_tile=32)
    y128 = ops.gemm_w4a4_fp4(codes, sfa, rs, pw, r.to(DEV), token_tile=128)
    _lib.device_status(0)
    ref = _fp4_reference(x, a.cpu(), w, r, fmt)
    err = ((y.double().cpu() - ref).abs().max() / ref.abs().max()).item()
    assert err < 1e-3, err
    assert torch.equal(y, y128)  # same tiles of K, same split, same order of sums
    with pytest.raises((RuntimeError, ValueError)):
        ops.gemm_w4a4_fp4(torch.cat([codes] * 40)[:33], sfa, None, pw, None, token_tile=32)


@pytest.mark.parametrize("fmt", [_lib.FP4_MXFP4, _lib.FP4_NVFP4])
@pytest.mark.parametrize("M,K", [(1, 256), (130, 512), (256, 1024), (37, 3584)])
def test_quantiser_writes_scale_factors_in_gemm_order(fmt, M, K):
    x = synthetic.make_x(M, K, M + K).to(DEV)
    a = torch.exp(torch.randn(K, generator=torch.Generator().manual_seed(K)) * 0.3).to(DEV)
    codes, sf, rs = ops.quant_fp4(x, fmt, a)
    codes2, sf_atoms, rs2 = ops.quant_fp4(x, fmt, a, atoms=True)
    assert torch.equal(codes, codes2)
    assert (rs is None and rs2 is None) or torch.equal(rs, rs2)
    # identical to the separate re-ordering pass, including the zero rows that pad the last tile
    assert torch.equal(sf_atoms, ops.fp4_sf_to_atoms(sf, K, fmt).reshape(-1))
