"""CPU oracle for the W4A4 hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this module;
the library itself never does.  Every function restates, in plain torch-on-CPU / numpy, the
arithmetic of one piece of the reference (sayehs-dmatrix/dualquant); the citation after each
name is the reference file:line it follows.

Parity status
-------------
* int4 path (activation quantiser, weight quantiser / packing, Hadamard, dequantise-and-matmul):
  pinned against the reference's own code, which is imported in the authoring container to
  produce the fixtures under tests/golden/ (see tests/golden/make_golden.py).
* MXFP4 / NVFP4 block casts: PARITY UNPINNED.  The reference delegates them to an external,
  non-redistributable package (`blockfmt` 0.3.0, formats/mx.py:24-29, formats/nvfp4.py:12-17)
  that is absent from the reference tree, and ships no test or golden vector at that boundary.
  The functions here follow the published OCP-MX / NVFP4 definitions and the in-tree statements
  of intent (legacy_vendor/torch_quant.py:326-375, scale_formats.py:23-45); the element
  rounding (`float_to_fp4`) *is* pinned against the reference.
"""
from __future__ import annotations

import math

import numpy as np
import torch

GROUP = 128


# ----------------------------------------------------------------------------------------------
# Hadamard matrices and transforms
# ----------------------------------------------------------------------------------------------
def _legendre(a: int, q: int) -> int:
    a %= q
    if a == 0:
        return 0
    return 1 if pow(a, (q - 1) // 2, q) == 1 else -1


def paley2_hadamard(q: int) -> torch.Tensor:
    """Paley type-II Hadamard matrix of order 2(q+1), q prime, q = 1 mod 4.

    With S the symmetric conference matrix [[0, 1^T], [1, Q]], Q[i][j] = legendre(j - i), the
    matrix is [[S + I, S - I], [S - I, -S - I]].  For q = 13 this is exactly the 28x28 literal
    of quarot/vendor/hadamard_utils.py:277-391 (`get_had28`); tests check that equality.
    """
    n = q + 1
    S = torch.zeros(n, n)
    S[0, 1:] = 1
    S[1:, 0] = 1
    for i in range(q):
        for j in range(q):
            S[1 + i, 1 + j] = _legendre(j - i, q)
    eye = torch.eye(n)
    top = torch.cat([S + eye, S - eye], dim=1)
    bot = torch.cat([S - eye, -S - eye], dim=1)
    return torch.cat([top, bot], dim=0).to(torch.float32)


_REFERENCE_ORDERS = (172, 156, 140, 108, 60, 52, 36, 28, 40, 20, 12)
_GOLDEN_HADAMARDS = {}


def reference_hadamard(k: int) -> torch.Tensor:
    """The k x k +-1 matrix of the reference's table (quarot/vendor/hadamard_utils.py:57-391), read
    from the fixture that tests/golden/make_golden.py produced by calling the reference's own
    get_had<k>() functions (one bit per entry)."""
    if not _GOLDEN_HADAMARDS:
        import os

        path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tests", "golden",
                            "reference_vectors.npz")
        blob = np.load(path)
        bits, off = blob["had_bits"], 0
        for order in blob["had_orders"].tolist():
            nbytes = (order * order + 7) // 8
            m = np.unpackbits(bits[off:off + nbytes])[: order * order].reshape(order, order)
            _GOLDEN_HADAMARDS[order] = torch.from_numpy(m.astype(np.float32) * 2 - 1)
            off += nbytes
    return _GOLDEN_HADAMARDS[k].clone()


def get_hadK(n: int):
    """(had_K, K) as the reference's get_hadK (quarot/vendor/hadamard_utils.py:5-55): the first order
    of its table that divides n, else (None, 1) for a power of two."""
    for k in _REFERENCE_ORDERS:
        if n % k == 0:
            assert _is_pow2(n // k)
            return reference_hadamard(k), k
    assert _is_pow2(n)
    return None, 1


def _is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


def wht_last_axis(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised Walsh-Hadamard butterflies along the last axis, stages h = 1, 2, 4, ...
    with (a, b) -> (a + b, a - b) (quarot/__init__.py:39-58).  Every output is formed by the same
    sequence of fp32 additions as the reference, so results are bit-identical."""
    n = x.shape[-1]
    assert _is_pow2(n)
    h = 1
    while h < n:
        y = x.reshape(x.shape[:-1] + (n // (2 * h), 2, h))
        a = y[..., 0, :]
        b = y[..., 1, :]
        x = torch.stack([a + b, a - b], dim=-2).reshape(x.shape[:-1] + (n,))
        h *= 2
    return x


def full_hadamard_scale(n: int) -> float:
    """The fp32 factor of hadamard_utils.py:97-99: 1.0 / torch.tensor(n).sqrt()."""
    return float((1.0 / torch.tensor(n).sqrt()).item())


def partial_hadamard_scale(num_heads: int) -> float:
    """perm_linear.py:96-98: python float 1/sqrt(H), applied to an fp32 tensor."""
    return float(np.float32(1.0 / math.sqrt(num_heads)))


def hadamard_full(x32: torch.Tensor, had_mat, had_k: int) -> torch.Tensor:
    """matmul_hadU_cuda (quarot/vendor/hadamard_utils.py:92-101) on fp32 rows [M, n].

    view(-1, K, n/K) -> WHT over the last axis -> * fp32 scale -> had_K @ .  The K x K stage is
    summed over j in ascending order in fp32 (the reference calls an fp32 matmul whose summation
    order is unspecified; codes derived from it may differ at exact rounding ties)."""
    M, n = x32.shape
    scale = torch.tensor(full_hadamard_scale(n), dtype=torch.float32)
    if had_k == 1:
        return wht_last_axis(x32) * scale
    v = wht_last_axis(x32.reshape(M, had_k, n // had_k)) * scale
    out = torch.zeros_like(v)
    for j in range(had_k):
        out = out + had_mat[:, j].reshape(1, had_k, 1) * v[:, j : j + 1, :]
    return out.reshape(M, n)


def hadamard_partial(x32: torch.Tensor, had_dim: int) -> torch.Tensor:
    """Online partial Hadamard of o_proj (activations/perm_linear.py:89-104, K == 1 branch):
    WHT across the head index for every head-dim lane, times 1/sqrt(H)."""
    M, n = x32.shape
    H = n // had_dim
    y = x32.reshape(M, H, had_dim).transpose(1, 2)
    y = wht_last_axis(y.contiguous()) * partial_hadamard_scale(H)
    return y.transpose(1, 2).reshape(M, n)


# ----------------------------------------------------------------------------------------------
# int4 quantisers
# ----------------------------------------------------------------------------------------------
def _round_scale_fp16(s: torch.Tensor) -> torch.Tensor:
    s16 = torch.clamp(s, max=65504.0).to(torch.float16).to(torch.float32)
    return torch.where(s16 == 0, torch.ones_like(s16), s16)


def quant_act_int4(x: torch.Tensor, a=None, had=None, scale_fp16: bool = False):
    """Per-token int4 quantiser: PermLinear._quantise_act (activations/perm_linear.py:108-134)
    with act_fmt = rtn_int4, block_size=-1 (formats/rtn_int.py:43-69).

    x: [M, K] bf16 (or fp32).  a: [K] fp32 or None.  had: None, ("full", had_mat, had_k) or
    ("partial", had_dim).  Returns (codes int8 [M,K], sx fp32 [M], x32 after scale + Hadamard).
    scale_fp16 rounds the token scale to fp16 before the division (the storage format the
    benchmark configuration names); False keeps the reference's fp32 scale."""
    x32 = x.to(torch.float32)
    if a is not None:
        x32 = x32 * a.to(torch.float32)
    if had is not None:
        if had[0] == "full":
            x32 = hadamard_full(x32, had[1], had[2])
        elif had[0] == "partial":
            x32 = hadamard_partial(x32, had[1])
        else:
            raise ValueError(had[0])
    amax = x32.abs().amax(dim=1, keepdim=True)
    s = amax / 7
    s[amax == 0] = 1.0
    if scale_fp16:
        s = _round_scale_fp16(s)
    q = (x32 / s).round().clamp(-8, 7)
    return q.to(torch.int8), s.reshape(-1).contiguous(), x32


def quant_act_int4_bf16_arith(x_bf16: torch.Tensor):
    """PermLinear._quantise_act without activation scale and Hadamard (activations/perm_linear.py:
    131-133): act_fmt.cast on the bf16 tensor itself, i.e. formats/rtn_int.py:62-67 evaluated by
    torch in bf16 (scale, quotient and product each rounded to bf16).
    Returns (codes int8 [M,K], scale as fp32 [M], de-quantised bf16 [M,K])."""
    assert x_bf16.dtype == torch.bfloat16
    xmax = x_bf16.abs().amax(dim=1, keepdim=True)
    s = xmax / 7
    s[xmax == 0] = 1.0
    q = (x_bf16 / s).round_().clamp_(-8, 7)
    return q.to(torch.int8), s.float().reshape(-1).contiguous(), q * s


def quant_act_int4_grouped(x: torch.Tensor, a=None, group: int = GROUP, scale_fp16: bool = False,
                           round_away: bool = False):
    """Activation quantiser with one scale per (token, K tile): the in-kernel quantiser of the
    reference's fused W4A4 Triton kernel (ablation/real_int4_kernel/fused_w4a4_kernel.py:93-100):
    a = x * beta in fp32, scale = absmax/7 per (row, tile) (1 where the tile is zero),
    q = clamp(round(a / scale), -8, 7) with libdevice.round (halves away from zero; round_away)
    or torch.round (halves to even, formats/rtn_int.py:67).
    Returns (codes int8 [M,K], scales fp32 [M, K/group])."""
    x32 = x.to(torch.float32)
    if a is not None:
        x32 = x32 * a.to(torch.float32)
    M, K = x32.shape
    xg = x32.reshape(M, K // group, group)
    amax = xg.abs().amax(dim=-1, keepdim=True)
    s = amax / 7
    s[amax == 0] = 1.0
    if scale_fp16:
        s = _round_scale_fp16(s)
    t = xg / s
    q = (torch.sign(t) * torch.floor(t.abs() + 0.5)) if round_away else t.round()
    q = q.clamp(-8, 7)
    return q.reshape(M, K).to(torch.int8), s.reshape(M, K // group).contiguous()


def epilogue_grouped(acc: torch.Tensor, sw: torch.Tensor, r, sxg: torch.Tensor, dtype=torch.float32):
    """fused_w4a4_kernel.py:119: acc += float(partial) * (a_scale * w_scale), groups in order;
    sxg is [M, K/group]; r[n] multiplies the finished sum."""
    M, N, G = acc.shape
    y = torch.zeros(M, N, dtype=dtype)
    for g in range(G):
        p = sxg[:, g].to(dtype).reshape(M, 1) * sw[:, g].to(dtype).reshape(1, N)
        y = y + acc[:, :, g].to(dtype) * p
    if r is not None:
        y = y * r.to(dtype).reshape(1, N)
    return y


def rmsnorm_bf16(x: torch.Tensor, weight=None, eps: float = 1e-5) -> torch.Tensor:
    """_RMSNbf16Safe.forward (quarot/llama_quarot.py:135-141): fp32 variance by .mean(-1),
    x * rsqrt(var + eps), cast back to the input dtype; with `weight` the HF LlamaRMSNorm form
    weight * normed.to(input_dtype), the product rounded in the input dtype."""
    x32 = x.to(torch.float32)
    var = x32.pow(2).mean(-1, keepdim=True)
    y = (x32 * torch.rsqrt(var + eps)).to(x.dtype)
    if weight is not None:
        y = weight.to(x.dtype) * y
    return y


def quant_w_int4(w: torch.Tensor, group: int = GROUP):
    """Symmetric per-group int4 weight quantiser (formats/rtn_int.py:43-69 with block_size =
    group; same grouping as pack_int4_weights, fused_dual_scale_kernel.py:156-189), with the
    group scale rounded to fp16 *before* the division so codes and stored scale agree.
    Returns (codes int8 [N,K], sw fp16 [N, K/group])."""
    N, K = w.shape
    wg = w.to(torch.float32).reshape(N, K // group, group)
    amax = wg.abs().amax(dim=-1, keepdim=True)
    s = amax / 7
    s[amax == 0] = 1.0
    s = _round_scale_fp16(s)
    q = (wg / s).round().clamp(-8, 7)
    return q.reshape(N, K).to(torch.int8), s.reshape(N, K // group).to(torch.float16)


def ref_pack_int4(codes: torch.Tensor) -> torch.Tensor:
    """The reference's packed layout (fused_dual_scale_kernel.py:179-186): unsigned code + 8,
    low nibble = even k, high nibble = odd k; uint8 [N, K/2]."""
    u = (codes.to(torch.int16) + 8).to(torch.uint8)
    return ((u[:, 0::2] & 0xF) | ((u[:, 1::2] & 0xF) << 4)).contiguous()


def ref_unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of ref_pack_int4 (dequant_int4_reference, fused_dual_scale_kernel.py:192-206,
    before the scale is applied)."""
    N, kh = packed.shape
    out = torch.empty(N, kh * 2, dtype=torch.int16)
    out[:, 0::2] = (packed & 0xF).to(torch.int16)
    out[:, 1::2] = ((packed >> 4) & 0xF).to(torch.int16)
    return (out - 8).to(torch.int8)


def stream_pack_int4(codes: torch.Tensor, sw: torch.Tensor, group: int = GROUP) -> torch.Tensor:
    """The library's streaming weight layout (flat uint8).  Tiles of 128 rows x 128 k in the order
    [row tile][k group]; a tile is 8192 bytes of codes ([row in tile][64 bytes]) followed by the
    128 fp16 group scales of its rows (256 bytes); rows past N are zero.  Within a tile row,
    k chunk ch covers k in [32ch, 32ch+32) of the group, its 16 bytes are
    byte b = (code[32ch+b] & 0xF) | ((code[32ch+16+b] & 0xF) << 4), two's complement nibbles,
    and it sits at chunk position ch ^ ((row_in_tile >> 1) & 3) of the 64-byte row."""
    N, K = codes.shape
    tiles, groups = (N + 127) // 128, K // group
    padded = torch.zeros(tiles * 128, K, dtype=torch.int16)
    padded[:N] = codes.to(torch.int16)
    c = padded.reshape(tiles, 128, groups, 4, 2, 16)
    lo = c[..., 0, :] & 0xF
    hi = c[..., 1, :] & 0xF
    byt = (lo | (hi << 4)).to(torch.uint8)  # [tiles, 128, groups, 4, 16]
    rows = torch.arange(128)
    src = torch.arange(4)[None, :] ^ ((rows >> 1) & 3)[:, None]  # [128, 4]: k chunk at each position
    idx = src.reshape(1, 128, 1, 4, 1).expand(tiles, 128, groups, 4, 16)
    byt = torch.gather(byt, 3, idx)  # position p of row r now holds k chunk p ^ ((r >> 1) & 3)
    body = byt.permute(0, 2, 1, 3, 4).contiguous().reshape(tiles, groups, 8192)
    scales = stream_pack_scales(sw).reshape(tiles, groups, 128).view(torch.uint8).reshape(tiles, groups, 256)
    return torch.cat([body, scales], dim=2).reshape(-1)


def stream_pack_scales(sw: torch.Tensor) -> torch.Tensor:
    """Group scales in the library's streaming order (flat fp16): [row tile][k group][row in
    tile], rows past N zero."""
    N, G = sw.shape
    tiles = (N + 127) // 128
    padded = torch.zeros(tiles * 128, G, dtype=torch.float16)
    padded[:N] = sw
    return padded.reshape(tiles, 128, G).permute(0, 2, 1).contiguous().reshape(-1)


# ----------------------------------------------------------------------------------------------
# GEMM
# ----------------------------------------------------------------------------------------------
def acc_int32(qx: torch.Tensor, qw: torch.Tensor, group: int = GROUP) -> torch.Tensor:
    """Exact per-group integer partial sums acc[m, n, g] = sum_{k in g} qx[m,k] * qw[n,k]
    (the int32 `tl.dot` of ablation/real_int4_kernel/fused_w4a4_kernel.py:116).  |acc| <= 8192,
    so an fp32 matmul per group is exact."""
    M, K = qx.shape
    N = qw.shape[0]
    G = K // group
    xa = qx.to(torch.float32).reshape(M, G, group).permute(1, 0, 2)
    wa = qw.to(torch.float32).reshape(N, G, group).permute(1, 2, 0)
    acc = torch.bmm(xa, wa)  # [G, M, N]
    return acc.permute(1, 2, 0).round().to(torch.int32).contiguous()


def epilogue(acc: torch.Tensor, sw: torch.Tensor, r, sx: torch.Tensor, dtype=torch.float32):
    """Y[m,n] = r[n] * sx[m] * sum_g sw[n,g] * acc[m,n,g]  (fused_w4a4_kernel.py:119 with one
    activation scale per token; r is the DualQuant row scale).  dtype float32 follows the
    kernel's order (groups ascending, then one scale product); float64 is the tie-breaker."""
    M, N, G = acc.shape
    swf = sw.to(dtype)
    run = torch.zeros(M, N, dtype=dtype)
    for g in range(G):
        run = run + acc[:, :, g].to(dtype) * swf[:, g].reshape(1, N)
    rr = torch.ones(N, dtype=dtype) if r is None else r.to(dtype)
    return run * (rr.reshape(1, N) * sx.to(dtype).reshape(M, 1))


def dequant_w(qw: torch.Tensor, sw: torch.Tensor, r=None, group: int = GROUP, dtype=torch.float32):
    """De-quantised weight diag(r) * (codes * group scale)  (dequant_int4_reference,
    fused_dual_scale_kernel.py:192-206)."""
    N, K = qw.shape
    w = qw.to(dtype).reshape(N, K // group, group) * sw.to(dtype).reshape(N, K // group, 1)
    w = w.reshape(N, K)
    if r is not None:
        w = w * r.to(dtype).reshape(N, 1)
    return w


def dequant_matmul(qx, sx, qw, sw, r=None, group: int = GROUP, dtype=torch.float64):
    """The reference's dequantise-and-matmul check (fused_dual_scale_kernel.py:287-292):
    (de-quantised activations) @ (de-quantised weights)^T."""
    xd = qx.to(dtype) * sx.to(dtype).reshape(-1, 1)
    return xd @ dequant_w(qw, sw, r, group, dtype).T


def perm_linear_fakequant(x, a, had, w_dq_bf16: torch.Tensor, scale_fp16: bool = False):
    """The reference's fake-quant forward (activations/perm_linear.py:136-141): de-quantised
    activations rounded to bf16, bf16 F.linear against the fake-quant weight."""
    q, s, _ = quant_act_int4(x, a, had, scale_fp16)
    xq = (q.to(torch.float32) * s.reshape(-1, 1)).to(torch.bfloat16)
    return torch.nn.functional.linear(xq, w_dq_bf16)


# ----------------------------------------------------------------------------------------------
# FP4 (parity unpinned except float_to_fp4 -- see the module docstring)
# ----------------------------------------------------------------------------------------------
_FP4_GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
_E4M3_TINY = 0.015625  # torch.finfo(torch.float8_e4m3fn).tiny = 2^-6


def float_to_fp4(x: torch.Tensor) -> torch.Tensor:
    """Round to the nearest E2M1 value, ties to the even mantissa, saturating at 6
    (legacy_vendor/torch_quant.py:326-356)."""
    ax = x.abs()
    out = torch.zeros_like(ax)
    out = torch.where(ax > 0.25, torch.full_like(ax, 0.5), out)
    out = torch.where(ax >= 0.75, torch.full_like(ax, 1.0), out)
    out = torch.where(ax > 1.25, torch.full_like(ax, 1.5), out)
    out = torch.where(ax >= 1.75, torch.full_like(ax, 2.0), out)
    out = torch.where(ax > 2.5, torch.full_like(ax, 3.0), out)
    out = torch.where(ax >= 3.5, torch.full_like(ax, 4.0), out)
    out = torch.where(ax > 5.0, torch.full_like(ax, 6.0), out)
    return torch.where(x < 0, -out, out)


def fp4_code(v: torch.Tensor) -> torch.Tensor:
    """E2M1 bit pattern (sign << 3 | magnitude index) of values already on the FP4 grid."""
    idx = torch.bucketize(v.abs().contiguous(), _FP4_GRID)
    idx = torch.clamp(idx, max=7)
    neg = (v < 0) | ((v == 0) & (torch.signbit(v)))
    return (idx | (neg.to(torch.int64) << 3)).to(torch.uint8)


# FP4 block formats ------------------------------------------------------------------------------
# MXFP4: blocks of 32 along the last axis, shared power-of-two scale (E8M0 byte = exponent + 127),
#        exponent = floor(log2(amax)) - 2 (2 = exponent of the largest E2M1 value 6 = 1.5 * 2^2),
#        as convert_to_mxfp (legacy_vendor/torch_quant.py:359-375); an all-zero block gets 2^-127.
# NVFP4: blocks of 16, E4M3 block scale on top of a second-level fp32 scale
#        ts = amax / (6 * 448) taken per token for activations or given per tensor for weights;
#        block scale = e4m3(clamp(amax_block / 6 / ts, 2^-6, 448)) (round to nearest; the clamp to
#        the normal E4M3 range is quantize_scale_e4m3's, scale_formats.py:39-45),
#        element = fp4(x / (ts * block scale)).
def _floor_log2(amax: torch.Tensor) -> torch.Tensor:
    bits = amax.contiguous().view(torch.int32)
    return ((bits >> 23) & 0xFF) - 127  # denormals report -127


def quant_mxfp4(x32: torch.Tensor, block: int = 32):
    """Returns (element values on the FP4 grid [.., K], E8M0 bytes [.., K/block], de-quantised)."""
    shape = x32.shape
    xb = x32.reshape(-1, shape[-1] // block, block)
    amax = xb.abs().amax(dim=-1)
    e = torch.where(amax == 0, torch.full_like(amax, -127, dtype=torch.int32), _floor_log2(amax) - 2)
    e = e.clamp(-127, 127)
    q = float_to_fp4(torch.ldexp(xb, (-e).unsqueeze(-1)))
    deq = torch.ldexp(q, e.unsqueeze(-1))
    return q.reshape(shape), (e + 127).to(torch.uint8).reshape(shape[:-1] + (-1,)), deq.reshape(shape)


def quant_nvfp4(x32: torch.Tensor, tensor_scale=None, block: int = 16):
    """Returns (FP4 element values, E4M3 block scales as fp32 [.., K/16], second-level scale
    [rows] fp32, de-quantised).  tensor_scale None -> one second-level scale per row."""
    shape = x32.shape
    x2 = x32.reshape(-1, shape[-1])
    if tensor_scale is None:
        amax_row = x2.abs().amax(dim=1, keepdim=True)
        ts = amax_row / 2688.0
        ts[amax_row == 0] = 1.0
    else:
        ts = torch.full((x2.shape[0], 1), float(tensor_scale), dtype=torch.float32)
    xb = x2.reshape(x2.shape[0], -1, block)
    amax = xb.abs().amax(dim=-1)
    bs = (amax / 6.0 / ts).clamp(min=_E4M3_TINY, max=448.0).to(torch.float8_e4m3fn).to(torch.float32)
    denom = (ts * bs).unsqueeze(-1)
    q = torch.where(denom == 0, torch.zeros_like(xb), float_to_fp4(xb / torch.where(denom == 0, torch.ones_like(denom), denom)))
    deq = q * bs.unsqueeze(-1) * ts.unsqueeze(-1)
    return q.reshape(shape), bs.reshape(shape[:-1] + (-1,)), ts.reshape(-1), deq.reshape(shape)


def pack_fp4(q: torch.Tensor) -> torch.Tensor:
    """Two E2M1 codes per byte, element 2j in the low nibble, 2j+1 in the high nibble."""
    c = fp4_code(q).reshape(q.shape[:-1] + (q.shape[-1] // 2, 2))
    return (c[..., 0] | (c[..., 1] << 4)).to(torch.uint8)


def e4m3_byte(v: torch.Tensor) -> torch.Tensor:
    return v.to(torch.float8_e4m3fn).view(torch.uint8)
