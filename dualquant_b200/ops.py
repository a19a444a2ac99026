"""Tensor-level wrappers over the C ABI: torch supplies device memory and the stream, the
shared library does all the work."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

GROUP = 128


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(dev: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _prep(t: torch.Tensor):
    if not t.is_cuda:
        raise RuntimeError("dualquant_b200 runs on CUDA (sm_100a) tensors only; got a CPU tensor")
    idx = t.device.index if t.device.index is not None else torch.cuda.current_device()
    if torch.cuda.current_device() != idx:
        torch.cuda.set_device(idx)
    _lib.ensure_init(idx)
    return _lib.load()


@dataclass
class Hadamard:
    """Online Hadamard description (the had_K / K / had_dim attributes of a PermLinear)."""

    kind: int = _lib.HAD_NONE
    had_k: int = 1
    had_dim: int = 0
    scale: float = 1.0
    had_mat: Optional[torch.Tensor] = None  # fp32 [had_k, had_k] on the device

    def desc(self):
        if self.kind == _lib.HAD_NONE:
            return None
        d = _lib.HadamardDesc()
        d.kind, d.had_k, d.had_dim, d.scale = self.kind, self.had_k, self.had_dim, self.scale
        d.had_mat = self.had_mat.data_ptr() if self.had_mat is not None else None
        return ctypes.byref(d)


@dataclass
class PackedInt4Weight:
    """Weight artefact the GEMM consumes: streaming int4 layout + transposed fp16 group scales."""

    w_packed: torch.Tensor  # uint8, flat: [row tile][k group][8192 B codes + 256 B scales]
    sw_t: torch.Tensor  # fp16, flat: [row tile][k group][128 rows]
    N: int
    K: int
    group: int = GROUP

    w8: Optional[torch.Tensor] = None  # derived E4M3 byte copy [N, K] for the prefill GEMM (not saved)

    def state(self):
        return {"w_packed": self.w_packed, "sw_t": self.sw_t, "N": self.N, "K": self.K,
                "group": self.group, "layout_version": 2}

    def bytes_e4m3(self) -> torch.Tensor:
        """The E4M3 byte form of the weight, expanded on first use and kept (N * K bytes)."""
        if self.w8 is None:
            self.w8 = expand_w_e4m3(self)
        return self.w8


def quant_w_int4(w: torch.Tensor, group: int = GROUP):
    """bf16 [N,K] -> (codes int8 [N,K], sw fp16 [N,K/group])."""
    lib = _prep(w)
    w = w.to(torch.bfloat16).contiguous()
    N, K = w.shape
    codes = torch.empty(N, K, dtype=torch.int8, device=w.device)
    sw = torch.empty(N, K // group, dtype=torch.float16, device=w.device)
    _lib.check(lib.dq_quant_w_int4(_ptr(w), N, K, group, _ptr(codes), _ptr(sw), _stream(w.device)),
               "dq_quant_w_int4")
    return codes, sw


def pack_w_int4(codes: Optional[torch.Tensor], sw: torch.Tensor, group: int = GROUP,
                ref_packed: Optional[torch.Tensor] = None) -> PackedInt4Weight:
    src = codes if codes is not None else ref_packed
    lib = _prep(src)
    if codes is not None:
        codes = codes.contiguous()
        N, K = codes.shape
    else:
        ref_packed = ref_packed.contiguous()
        N, K = ref_packed.shape[0], ref_packed.shape[1] * 2
    sw = sw.to(torch.float16).contiguous()
    w_packed = torch.empty(int(lib.dq_packed_w_bytes(N, K)), dtype=torch.uint8, device=src.device)
    sw_t = torch.empty((N + 127) // 128 * 128 * (K // group), dtype=torch.float16, device=src.device)
    _lib.check(lib.dq_pack_w_int4(_ptr(codes), _ptr(ref_packed), _ptr(sw), N, K, group, _ptr(w_packed),
                                  _ptr(sw_t), _stream(src.device)), "dq_pack_w_int4")
    return PackedInt4Weight(w_packed, sw_t, N, K, group)


def unpack_w_int4(pw: PackedInt4Weight) -> torch.Tensor:
    lib = _prep(pw.w_packed)
    codes = torch.empty(pw.N, pw.K, dtype=torch.int8, device=pw.w_packed.device)
    _lib.check(lib.dq_unpack_w_int4(_ptr(pw.w_packed), pw.N, pw.K, _ptr(codes),
                                    _stream(codes.device)), "dq_unpack_w_int4")
    return codes


def _scale_mode(scale_fp16: bool, bf16_arith: bool) -> int:
    """The C ABI's scale_fp16 argument: 0 = fp32 token scale, 1 = rounded to fp16, 2 = the whole
    quantiser in bf16 arithmetic (the reference's path without activation scale and Hadamard)."""
    if bf16_arith and scale_fp16:
        raise ValueError("bf16 arithmetic and an fp16 token scale exclude each other")
    return 2 if bf16_arith else int(bool(scale_fp16))


def quant_act_int4(x: torch.Tensor, a: Optional[torch.Tensor] = None,
                   had: Optional[Hadamard] = None, scale_fp16: bool = False, bf16_arith: bool = False,
                   e4m3: bool = False):
    """bf16 or fp32 [M,K] -> (codes int8 [M,K], sx fp32 [M]); e4m3: the codes as E4M3 bytes (uint8),
    the operand of gemm_w4a4_int4_e4m3."""
    lib = _prep(x)
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("quant_act_int4 expects bf16 or fp32 activations")
    if x.stride(-1) != 1:
        x = x.contiguous()
    M, K = x.shape
    codes = torch.empty(M, K, dtype=torch.uint8 if e4m3 else torch.int8, device=x.device)
    sx = torch.empty(M, dtype=torch.float32, device=x.device)
    desc = had.desc() if had is not None else None
    fn, what = ((lib.dq_quant_act_int4, "dq_quant_act_int4") if x.dtype == torch.bfloat16
                else (lib.dq_quant_act_int4_f32, "dq_quant_act_int4_f32"))
    _lib.check(fn(_ptr(x), x.stride(0) if M > 1 else K, _ptr(a), desc, M, K, _ptr(codes), _ptr(sx),
                  _scale_mode(scale_fp16, bf16_arith) | (_lib.CODES_E4M3 if e4m3 else 0), _stream(x.device)), what)
    return codes, sx


def quant_act_int4_gated(gate: torch.Tensor, up: torch.Tensor, a: Optional[torch.Tensor] = None,
                         had: Optional[Hadamard] = None, scale_fp16: bool = False, e4m3: bool = False):
    """codes/scales of bf16(bf16(SiLU(gate)) * up); gate and up are bf16 [M,K] views with the same
    row stride (typically the two halves of a fused gate+up projection output)."""
    lib = _prep(gate)
    if gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16:
        raise ValueError("quant_act_int4_gated expects bf16 inputs")
    if gate.shape != up.shape or gate.stride() != up.stride() or gate.stride(-1) != 1:
        raise ValueError("gate and up must have the same shape and strides (unit inner stride)")
    M, K = gate.shape
    codes = torch.empty(M, K, dtype=torch.uint8 if e4m3 else torch.int8, device=gate.device)
    sx = torch.empty(M, dtype=torch.float32, device=gate.device)
    desc = had.desc() if had is not None else None
    _lib.check(lib.dq_quant_act_int4_gated(_ptr(gate), _ptr(up), gate.stride(0) if M > 1 else K, _ptr(a),
                                           desc, M, K, _ptr(codes), _ptr(sx),
                                           int(scale_fp16) | (_lib.CODES_E4M3 if e4m3 else 0),
                                           _stream(gate.device)), "dq_quant_act_int4_gated")
    return codes, sx


def quant_act_int4_rmsnorm(x: torch.Tensor, norm_weight: Optional[torch.Tensor], eps: float,
                           a: Optional[torch.Tensor] = None, scale_fp16: bool = False, e4m3: bool = False):
    """RMSNorm (bf16 result, optional bf16 weight) + column scale + per-token int4 quantiser in
    one pass: bf16 [M,K] -> (codes int8 [M,K], sx fp32 [M])."""
    lib = _prep(x)
    if x.dtype != torch.bfloat16 or x.stride(-1) != 1:
        raise ValueError("quant_act_int4_rmsnorm expects bf16 rows with unit inner stride")
    if norm_weight is not None and (norm_weight.dtype != torch.bfloat16 or norm_weight.numel() != x.shape[1]):
        raise ValueError("norm_weight must be bf16 with one entry per input channel")
    M, K = x.shape
    codes = torch.empty(M, K, dtype=torch.uint8 if e4m3 else torch.int8, device=x.device)
    sx = torch.empty(M, dtype=torch.float32, device=x.device)
    _lib.check(lib.dq_quant_act_int4_rmsnorm(_ptr(x), x.stride(0) if M > 1 else K, _ptr(norm_weight),
                                             float(eps), _ptr(a), M, K, _ptr(codes), _ptr(sx),
                                             int(scale_fp16) | (_lib.CODES_E4M3 if e4m3 else 0), _stream(x.device)),
               "dq_quant_act_int4_rmsnorm")
    return codes, sx


def fakequant_act_int4(x: torch.Tensor, a: Optional[torch.Tensor] = None,
                       had: Optional[Hadamard] = None, scale_fp16: bool = False,
                       bf16_arith: bool = False) -> torch.Tensor:
    """[M,K] bf16 or fp32 -> de-quantised fp32 [M,K] (what FormatSpec.cast returns)."""
    lib = _prep(x)
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("fakequant_act_int4 expects bf16 or fp32")
    x = x.contiguous()
    M, K = x.shape
    out = torch.empty(M, K, dtype=torch.float32, device=x.device)
    desc = had.desc() if had is not None else None
    _lib.check(lib.dq_fakequant_act_int4(_ptr(x), int(x.dtype == torch.float32), K, _ptr(a), desc,
                                         M, K, _ptr(out), _scale_mode(scale_fp16, bf16_arith),
                                         _stream(x.device)),
               "dq_fakequant_act_int4")
    return out


def hadamard_f32(x: torch.Tensor, had: Hadamard) -> torch.Tensor:
    lib = _prep(x)
    x = x.to(torch.float32).contiguous()
    M, K = x.shape
    out = torch.empty_like(x)
    _lib.check(lib.dq_hadamard_f32(_ptr(x), _ptr(out), M, K, had.desc(), _stream(x.device)),
               "dq_hadamard_f32")
    return out


def quant_act_int4_grouped(x: torch.Tensor, a: Optional[torch.Tensor] = None, scale_fp16: bool = False,
                           round_away: bool = False):
    """bf16 [M,K] -> (codes int8 [M,K], scales fp32 [K/128, M]): one activation scale per (token,
    group of 128), the quantiser of the reference's fused W4A4 Triton kernel."""
    lib = _prep(x)
    if x.dtype != torch.bfloat16:
        raise ValueError("quant_act_int4_grouped expects bf16 activations")
    if x.stride(-1) != 1:
        x = x.contiguous()
    M, K = x.shape
    codes = torch.empty(M, K, dtype=torch.int8, device=x.device)
    sxg = torch.empty(K // GROUP, M, dtype=torch.float32, device=x.device)
    _lib.check(lib.dq_quant_act_int4_grouped(_ptr(x), x.stride(0) if M > 1 else K, _ptr(a), M, K, GROUP,
                                             _ptr(codes), _ptr(sxg), int(scale_fp16), int(round_away),
                                             _stream(x.device)), "dq_quant_act_int4_grouped")
    return codes, sxg


def gemm_w4a4_int4_grouped(codes: torch.Tensor, sxg: torch.Tensor, pw: PackedInt4Weight,
                           r: Optional[torch.Tensor] = None, out_dtype=torch.float32) -> torch.Tensor:
    """The int4 GEMM with per-(token, group) activation scales sxg [K/128, M]."""
    lib = _prep(codes)
    M, K = codes.shape
    if K != pw.K or tuple(sxg.shape) != (K // pw.group, M):
        raise ValueError("shape mismatch between codes, group scales and weight")
    out = torch.empty(M, pw.N, dtype=out_dtype, device=codes.device)
    ydt = _lib.DTYPE_BF16 if out.dtype == torch.bfloat16 else _lib.DTYPE_F32
    _lib.check(lib.dq_gemm_w4a4_int4_grouped(_ptr(codes), _ptr(sxg.contiguous()), _ptr(pw.w_packed),
                                             _ptr(pw.sw_t), _ptr(r), M, pw.N, K, pw.group, _ptr(out), ydt,
                                             _stream(codes.device)), "dq_gemm_w4a4_int4_grouped")
    return out


def fakequant_act_int4_bf16(x: torch.Tensor) -> torch.Tensor:
    """bf16 [M,K] -> bf16 [M,K]: per-token int4 fake-quantisation in one pass (the
    quantize_bmm_input step of PermLinear)."""
    lib = _prep(x)
    if x.dtype != torch.bfloat16:
        raise ValueError("fakequant_act_int4_bf16 expects bf16 rows")
    if x.stride(-1) != 1:
        x = x.contiguous()
    M, K = x.shape
    out = torch.empty(M, K, dtype=torch.bfloat16, device=x.device)
    _lib.check(lib.dq_fakequant_act_int4_bf16(_ptr(x), x.stride(0) if M > 1 else K, M, K, _ptr(out),
                                              _stream(x.device)), "dq_fakequant_act_int4_bf16")
    return out


def gemm_w4a4_int4(codes: torch.Tensor, sx: torch.Tensor, pw: PackedInt4Weight,
                   r: Optional[torch.Tensor] = None, out_dtype=torch.float32,
                   token_tile: int = 0, split_k: int = 0,
                   out: Optional[torch.Tensor] = None,
                   residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual: [M, N] of the output's dtype -> out = residual + linear (fused into the epilogue;
    may be the output tensor itself)."""
    lib = _prep(codes)
    M, K = codes.shape
    if K != pw.K:
        raise ValueError(f"K mismatch: activations {K}, weight {pw.K}")
    if out is None:
        out = torch.empty(M, pw.N, dtype=residual.dtype if residual is not None else out_dtype,
                          device=codes.device)
    ydt = _lib.DTYPE_BF16 if out.dtype == torch.bfloat16 else _lib.DTYPE_F32
    if residual is not None:
        if residual.dtype != out.dtype or tuple(residual.shape) != (M, pw.N) or not residual.is_contiguous():
            raise ValueError("residual must be a contiguous [M, N] tensor of the output's dtype")
        _lib.check(lib.dq_gemm_w4a4_int4_residual(_ptr(codes), _ptr(sx), _ptr(pw.w_packed), _ptr(pw.sw_t),
                                                  _ptr(r), _ptr(residual), M, pw.N, K, pw.group, _ptr(out),
                                                  ydt, _stream(codes.device)), "dq_gemm_w4a4_int4_residual")
        return out
    _lib.check(lib.dq_gemm_w4a4_int4_ex(_ptr(codes), _ptr(sx), _ptr(pw.w_packed), _ptr(pw.sw_t), _ptr(r),
                                        M, pw.N, K, pw.group, _ptr(out), ydt, None, 0,
                                        _stream(codes.device), token_tile, split_k),
               "dq_gemm_w4a4_int4")
    return out


def expand_w_e4m3(pw: PackedInt4Weight) -> torch.Tensor:
    """E4M3 byte copy [N, K] of the packed int4 weight (operand of gemm_w4a4_int4_e4m3)."""
    lib = _prep(pw.w_packed)
    w8 = torch.empty(pw.N, pw.K, dtype=torch.uint8, device=pw.w_packed.device)
    _lib.check(lib.dq_expand_w_int4_e4m3(_ptr(pw.w_packed), pw.N, pw.K, pw.group, _ptr(w8),
                                         _stream(w8.device)), "dq_expand_w_int4_e4m3")
    return w8


def codes_to_e4m3(codes: torch.Tensor) -> torch.Tensor:
    """int8 activation codes [M, K] -> the same integers as E4M3 bytes."""
    lib = _prep(codes)
    M, K = codes.shape
    x8 = torch.empty(M, K, dtype=torch.uint8, device=codes.device)
    _lib.check(lib.dq_codes_to_e4m3(_ptr(codes), codes.stride(0), M, K, _ptr(x8), _stream(codes.device)),
               "dq_codes_to_e4m3")
    return x8


def gemm_w4a4_int4_e4m3(x8: torch.Tensor, sx: torch.Tensor, w8: torch.Tensor, pw: PackedInt4Weight,
                        r: Optional[torch.Tensor] = None, out_dtype=torch.float32,
                        out: Optional[torch.Tensor] = None,
                        residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The int4 GEMM on the FP8 tensor-core path (prefill); same bits as gemm_w4a4_int4."""
    lib = _prep(x8)
    M, K = x8.shape
    if K != pw.K or tuple(w8.shape) != (pw.N, pw.K) or not x8.is_contiguous() or not w8.is_contiguous():
        raise ValueError("x8 [M, K] and w8 [N, K] must be contiguous and match the packed weight")
    if out is None:
        out = torch.empty(M, pw.N, dtype=residual.dtype if residual is not None else out_dtype, device=x8.device)
    if residual is not None and (residual.dtype != out.dtype or tuple(residual.shape) != (M, pw.N)
                                 or not residual.is_contiguous()):
        raise ValueError("residual must be a contiguous [M, N] tensor of the output's dtype")
    ydt = _lib.DTYPE_BF16 if out.dtype == torch.bfloat16 else _lib.DTYPE_F32
    _lib.check(lib.dq_gemm_w4a4_int4_e4m3(_ptr(x8), _ptr(sx), _ptr(w8), _ptr(pw.sw_t), _ptr(r), M, pw.N, K,
                                          pw.group, _ptr(out), ydt, _ptr(residual), _stream(x8.device)),
               "dq_gemm_w4a4_int4_e4m3")
    return out


class AllReduceContext:
    """Peer-mapped exchange buffers of the all-reduce fused into the decode GEMM
    (dq_gemm_w4a4_int4_ar).  Built once per process group from torch symmetric memory: one
    allocation per rank holding 2 * capacity fp32 (double-buffered partial outputs) followed by
    the flag array; every rank maps every other rank's allocation over NVLink.  All ranks must
    construct it collectively and then issue the same sequence of gemm_w4a4_int4_ar calls."""

    FLAG_UNITS = 1024

    def __init__(self, group, device, capacity_floats: int = 16 * 16384):
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("the fused all-reduce covers one NVLink domain of at most 8 ranks")
        cap = (int(capacity_floats) + 63) // 64 * 64
        words = 2 * cap + self.FLAG_UNITS * 8
        self._mem = symm.empty(words, dtype=torch.float32, device=device)
        self._mem.zero_()
        self._handle = symm.rendezvous(self._mem, group)
        self.seq = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group, device_ids=[device.index])  # every rank's flags are zero from here on
        ctx = _lib.AllReduceCtx()
        ctx.world, ctx.rank = self.world, self.rank
        for p in range(self.world):
            base = int(self._handle.buffer_ptrs[p])
            ctx.buf_ptrs[p] = base
            ctx.flag_ptrs[p] = base + 2 * cap * 4
        ctx.seq = self.seq.data_ptr()
        ctx.buf_capacity_floats = cap
        ctx.flag_units = self.FLAG_UNITS
        self.capacity = cap
        self._ctx = ctx
        self._ref = ctypes.byref(ctx)


def gemm_w4a4_int4_ar(codes: torch.Tensor, sx: torch.Tensor, pw: PackedInt4Weight,
                      r: Optional[torch.Tensor], ctx: AllReduceContext, out_dtype=torch.float32,
                      out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-parallel int4 GEMM of a decode batch (M <= 16): this rank's K slice, summed over the
    ranks of `ctx` inside the kernel; every rank gets the full [M, N] result (+ residual [M, N] of
    the output's dtype, added as the sum is stored)."""
    lib = _prep(codes)
    M, K = codes.shape
    if K != pw.K:
        raise ValueError(f"K mismatch: activations {K}, weight {pw.K}")
    if out is None:
        out = torch.empty(M, pw.N, dtype=residual.dtype if residual is not None else out_dtype, device=codes.device)
    if residual is not None and (residual.dtype != out.dtype or tuple(residual.shape) != (M, pw.N)
                                 or not residual.is_contiguous()):
        raise ValueError("residual must be a contiguous [M, N] tensor of the output's dtype")
    ydt = _lib.DTYPE_BF16 if out.dtype == torch.bfloat16 else _lib.DTYPE_F32
    _lib.check(lib.dq_gemm_w4a4_int4_ar_residual(_ptr(codes), _ptr(sx), _ptr(pw.w_packed), _ptr(pw.sw_t), _ptr(r),
                                                 _ptr(residual), M, pw.N, K, pw.group, _ptr(out), ydt,
                                                 _stream(codes.device), ctx._ref), "dq_gemm_w4a4_int4_ar_residual")
    return out


class ExchangeContext:
    """Peer-mapped buffers of the token-sharded prompt pass under tensor parallelism (one allocation
    per rank in torch symmetric memory, every rank maps all of them): partial outputs
    [world][tokens_per_rank][hidden] bf16, gathered activation codes [world * tokens_per_rank][hidden]
    bytes, gathered token scales, barrier words.  Built collectively; afterwards all ranks must issue
    the same sequence of exchange calls (every rank counts its barriers on the device)."""

    def __init__(self, group, device, tokens_per_rank: int, hidden: int):
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("the exchange covers one NVLink domain of at most 8 ranks")
        if tokens_per_rank % 256 or hidden % 128:
            raise ValueError("tokens_per_rank must be a multiple of 256 and hidden a multiple of 128")
        self.tokens_per_rank, self.hidden = int(tokens_per_rank), int(hidden)
        T = self.world * self.tokens_per_rank
        part_b = T * hidden * 2
        codes_b = T * hidden
        sx_b = (T * 4 + 255) // 256 * 256
        total = part_b + codes_b + sx_b + 256
        self._mem = symm.empty(total, dtype=torch.uint8, device=device)
        self._mem[part_b + codes_b + sx_b:].zero_()
        self._handle = symm.rendezvous(self._mem, group)
        torch.cuda.synchronize(device)
        dist.barrier(group=group, device_ids=[device.index])  # every rank's barrier words are zero from here on
        ctx = _lib.ExchangeCtx()
        ctx.world, ctx.rank = self.world, self.rank
        for p in range(self.world):
            base = int(self._handle.buffer_ptrs[p])
            ctx.part_ptrs[p] = base
            ctx.codes_ptrs[p] = base + part_b
            ctx.sx_ptrs[p] = base + part_b + codes_b
            ctx.flag_ptrs[p] = base + part_b + codes_b + sx_b
        ctx.tokens_per_rank, ctx.hidden = self.tokens_per_rank, self.hidden
        self._count = torch.zeros(1, dtype=torch.int32, device=device)  # this rank's barriers so far
        ctx.barrier_count = self._count.data_ptr()
        self._ctx = ctx
        self._ref = ctypes.byref(ctx)
        # this rank's views of its own buffers
        self.part = self._mem[:part_b].view(torch.bfloat16).view(self.world, self.tokens_per_rank, hidden)
        self.codes = self._mem[part_b:part_b + codes_b].view(T, hidden)
        self.sx = self._mem[part_b + codes_b:part_b + codes_b + T * 4].view(torch.float32)

    def barrier(self):
        """Device-side barrier across the ranks on the current stream (bounded wait).  The epoch is
        counted on the device, so the call can sit in a captured CUDA graph."""
        lib = _prep(self._mem)
        _lib.check(lib.dq_exchange_barrier(self._ref, 0, _stream(self._mem.device)), "dq_exchange_barrier")

    def add_partials(self, x: torch.Tensor):
        """x [tokens_per_rank, hidden] bf16 += the ranks' partial rows for this rank's tokens."""
        lib = _prep(x)
        if x.dtype != torch.bfloat16 or tuple(x.shape) != (self.tokens_per_rank, self.hidden) or not x.is_contiguous():
            raise ValueError("x must be a contiguous bf16 [tokens_per_rank, hidden] tensor")
        _lib.check(lib.dq_exchange_sum(self._ref, _ptr(x), _stream(x.device)), "dq_exchange_sum")

    def push(self, codes: torch.Tensor, sx: torch.Tensor):
        """This rank's codes [tokens_per_rank, hidden] (E4M3 bytes) and token scales into every rank's
        gathered buffers."""
        lib = _prep(codes)
        if (codes.dtype != torch.uint8 or tuple(codes.shape) != (self.tokens_per_rank, self.hidden)
                or not codes.is_contiguous() or sx.dtype != torch.float32 or sx.numel() != self.tokens_per_rank):
            raise ValueError("codes must be uint8 [tokens_per_rank, hidden], sx fp32 [tokens_per_rank]")
        _lib.check(lib.dq_exchange_push(self._ref, _ptr(codes), _ptr(sx), _stream(codes.device)), "dq_exchange_push")


def gemm_w4a4_int4_e4m3_scatter(x8: torch.Tensor, sx: torch.Tensor, w8: torch.Tensor, pw: PackedInt4Weight,
                                r: Optional[torch.Tensor], ctx: ExchangeContext) -> None:
    """Row-parallel int4 GEMM of the token-sharded prompt pass: this rank's K slice; the bf16 output
    tiles go from the kernel's epilogue into the partial buffer of the rank that owns the tokens."""
    lib = _prep(x8)
    M, K = x8.shape
    if K != pw.K or tuple(w8.shape) != (pw.N, pw.K) or not x8.is_contiguous() or not w8.is_contiguous():
        raise ValueError("x8 [M, K] and w8 [N, K] must be contiguous and match the packed weight")
    _lib.check(lib.dq_gemm_w4a4_int4_e4m3_scatter(_ptr(x8), _ptr(sx), _ptr(w8), _ptr(pw.sw_t), _ptr(r), M, pw.N, K,
                                                  pw.group, ctx._ref, _stream(x8.device)),
               "dq_gemm_w4a4_int4_e4m3_scatter")


def gemm_w4a4_int4_acc(codes: torch.Tensor, pw: PackedInt4Weight) -> torch.Tensor:
    """Test hook: raw per-group int32 accumulators [M, N, K/G]."""
    lib = _prep(codes)
    M, K = codes.shape
    acc = torch.zeros(M, pw.N, K // pw.group, dtype=torch.int32, device=codes.device)
    _lib.check(lib.dq_gemm_w4a4_int4_acc(_ptr(codes), _ptr(pw.w_packed), M, pw.N, K, pw.group,
                                         _ptr(acc), _stream(codes.device)), "dq_gemm_w4a4_int4_acc")
    return acc


def linear_scratch_bytes(M: int, N: int, K: int, prefill: bool = True) -> int:
    """Scratch of linear_w4a4_int4; prefill=True includes the room that lets batches of 1024 tokens
    and more take the FP8-path GEMM (N * K bytes more for those, nothing for smaller batches)."""
    lib = _lib.load()
    if prefill:
        return int(lib.dq_linear_w4a4_int4_prefill_scratch_bytes(M, N, K))
    return int(lib.dq_linear_w4a4_int4_scratch_bytes(M, N, K))


def linear_w4a4_int4(x: torch.Tensor, a: Optional[torch.Tensor], had: Optional[Hadamard],
                     pw: PackedInt4Weight, r: Optional[torch.Tensor], out_dtype=torch.float32,
                     scale_fp16: bool = False, scratch: Optional[torch.Tensor] = None,
                     out: Optional[torch.Tensor] = None, bf16_arith: bool = False) -> torch.Tensor:
    """Whole PermLinear.forward on the int4 path in one C call."""
    lib = _prep(x)
    if x.dtype != torch.bfloat16:
        raise ValueError("linear_w4a4_int4 expects bf16 activations (quantise fp32 rows with "
                         "quant_act_int4 and call gemm_w4a4_int4)")
    if x.stride(-1) != 1:
        x = x.contiguous()
    M, K = x.shape
    # a caller's scratch is used as it is when it covers the plain path; the C side takes the
    # FP8-path GEMM for prefill batches only if the scratch also has room for the weight's byte form
    if scratch is None or scratch.numel() < linear_scratch_bytes(M, pw.N, K, prefill=False):
        scratch = torch.empty(max(linear_scratch_bytes(M, pw.N, K), 256), dtype=torch.uint8, device=x.device)
    if out is None:
        out = torch.empty(M, pw.N, dtype=out_dtype, device=x.device)
    ydt = _lib.DTYPE_BF16 if out.dtype == torch.bfloat16 else _lib.DTYPE_F32
    desc = had.desc() if had is not None else None
    _lib.check(lib.dq_linear_w4a4_int4(_ptr(x), x.stride(0) if M > 1 else K, _ptr(a), desc,
                                       _ptr(pw.w_packed), _ptr(pw.sw_t), _ptr(r), M, pw.N, K, pw.group,
                                       _ptr(out), ydt, _scale_mode(scale_fp16, bf16_arith), _ptr(scratch),
                                       scratch.numel(), _stream(x.device)), "dq_linear_w4a4_int4")
    return out


def linear_a16w4(x: torch.Tensor, a: Optional[torch.Tensor], pw: PackedInt4Weight,
                 r: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16,
                 scratch: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 activations (times the column scale a, rounded to fp16) against the int4 weight
    artefact on the 16-bit tensor cores: Y = r * (fp16(x * a) @ fp16(codes * group scale)^T)."""
    lib = _prep(x)
    if x.dtype != torch.bfloat16:
        raise ValueError("linear_a16w4 expects bf16 activations")
    if x.stride(-1) != 1:
        x = x.contiguous()
    M, K = x.shape
    if K != pw.K:
        raise ValueError(f"K mismatch: activations {K}, weight {pw.K}")
    need = int(lib.dq_linear_a16w4_scratch_bytes(M, pw.N, K))
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(max(need, 256), dtype=torch.uint8, device=x.device)
    if out is None:
        out = torch.empty(M, pw.N, dtype=out_dtype, device=x.device)
    ydt = _lib.DTYPE_BF16 if out.dtype == torch.bfloat16 else _lib.DTYPE_F32
    _lib.check(lib.dq_linear_a16w4(_ptr(x), x.stride(0) if M > 1 else K, _ptr(a), _ptr(pw.w_packed), _ptr(r),
                                   M, pw.N, K, pw.group, _ptr(out), ydt, _ptr(scratch),
                                   0 if scratch is None else scratch.numel(), _stream(x.device)),
               "dq_linear_a16w4")
    return out


# ---------------------------------------------------------------------------------------------
# block-scaled FP4
# ---------------------------------------------------------------------------------------------
def _fp4_block(fmt: int) -> int:
    return 32 if fmt == _lib.FP4_MXFP4 else 16


def quant_fp4(x: torch.Tensor, fmt: int, a: Optional[torch.Tensor] = None,
              tensor_scale: Optional[torch.Tensor] = None, atoms: bool = False):
    """[M,K] bf16/fp32 -> (codes uint8 [M,K/2], sf uint8 [M,K/block], row_scale fp32 [M] or None).
    atoms=True: the scale bytes come back flat, already in the order the GEMM streams."""
    lib = _prep(x)
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("quant_fp4 expects bf16 or fp32")
    x = x.contiguous()
    M, K = x.shape
    codes = torch.empty(M, K // 2, dtype=torch.uint8, device=x.device)
    row_scale = None
    if fmt == _lib.FP4_NVFP4 and tensor_scale is None:
        row_scale = torch.empty(M, dtype=torch.float32, device=x.device)
    if atoms:
        sf = torch.empty(int(lib.dq_fp4_sf_atoms_bytes(M, K, fmt)), dtype=torch.uint8, device=x.device)
        _lib.check(lib.dq_quant_fp4_atoms(_ptr(x), int(x.dtype == torch.float32), K, _ptr(a), M, K, fmt,
                                          _ptr(tensor_scale), _ptr(codes), _ptr(sf), _ptr(row_scale),
                                          _stream(x.device)), "dq_quant_fp4_atoms")
        return codes, sf, row_scale
    sf = torch.empty(M, K // _fp4_block(fmt), dtype=torch.uint8, device=x.device)
    _lib.check(lib.dq_quant_fp4(_ptr(x), int(x.dtype == torch.float32), K, _ptr(a), M, K, fmt,
                                _ptr(tensor_scale), _ptr(codes), _ptr(sf), _ptr(row_scale),
                                _stream(x.device)), "dq_quant_fp4")
    return codes, sf, row_scale


def fakequant_fp4(x: torch.Tensor, fmt: int, a: Optional[torch.Tensor] = None,
                  tensor_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = _prep(x)
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("fakequant_fp4 expects bf16 or fp32")
    x = x.contiguous()
    M, K = x.shape
    out = torch.empty(M, K, dtype=torch.float32, device=x.device)
    _lib.check(lib.dq_fakequant_fp4(_ptr(x), int(x.dtype == torch.float32), K, _ptr(a), M, K, fmt,
                                    _ptr(tensor_scale), _ptr(out), _stream(x.device)),
               "dq_fakequant_fp4")
    return out


def nvfp4_tensor_scale(x: torch.Tensor) -> torch.Tensor:
    """absmax(x) / (6 * 448) as a one-element device tensor (1 for an all-zero tensor)."""
    lib = _prep(x)
    x = x.contiguous()
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.float()
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    _lib.check(lib.dq_nvfp4_tensor_scale(_ptr(x), int(x.dtype == torch.float32), x.numel(), _ptr(scale),
                                         _stream(x.device)), "dq_nvfp4_tensor_scale")
    return scale


def fp4_sf_to_atoms(sf: torch.Tensor, K: int, fmt: int) -> torch.Tensor:
    lib = _prep(sf)
    rows = sf.shape[0]
    out = torch.empty(int(lib.dq_fp4_sf_atoms_bytes(rows, K, fmt)), dtype=torch.uint8, device=sf.device)
    _lib.check(lib.dq_fp4_sf_to_atoms(_ptr(sf.contiguous()), rows, K, fmt, _ptr(out), _stream(sf.device)),
               "dq_fp4_sf_to_atoms")
    return out


@dataclass
class PackedFp4Weight:
    """FP4 weight artefact: packed E2M1 codes, scale factors in GEMM order, NVFP4 tensor scale."""

    codes: torch.Tensor  # uint8 [N, K/2]
    sf_atoms: torch.Tensor  # uint8, flat
    tensor_scale: Optional[torch.Tensor]  # fp32 [1] (NVFP4) or None
    N: int
    K: int
    fmt: int


def pack_w_fp4(w: torch.Tensor, fmt: int) -> PackedFp4Weight:
    """bf16/fp32 [N,K] -> FP4 artefact (blocks along K; NVFP4 uses one per-tensor second-level scale)."""
    w = w.contiguous()
    if w.dtype not in (torch.bfloat16, torch.float32):
        w = w.float()
    N, K = w.shape
    ts = nvfp4_tensor_scale(w) if fmt == _lib.FP4_NVFP4 else None
    codes, sf, _ = quant_fp4(w, fmt, None, ts)
    return PackedFp4Weight(codes, fp4_sf_to_atoms(sf, K, fmt), ts, N, K, fmt)


def gemm_w4a4_fp4(x_codes: torch.Tensor, x_sf_atoms: torch.Tensor, x_scale: Optional[torch.Tensor],
                  pw: PackedFp4Weight, r: Optional[torch.Tensor] = None, out_dtype=torch.float32,
                  out: Optional[torch.Tensor] = None, token_tile: int = 0) -> torch.Tensor:
    """token_tile: 0 = library's choice, 32 / 128 / 256 tokens per CTA (256 has no split-K)."""
    lib = _prep(x_codes)
    M = x_codes.shape[0]
    if out is None:
        out = torch.empty(M, pw.N, dtype=out_dtype, device=x_codes.device)
    ydt = _lib.DTYPE_BF16 if out.dtype == torch.bfloat16 else _lib.DTYPE_F32
    _lib.check(lib.dq_gemm_w4a4_fp4_tiled(_ptr(x_codes), _ptr(x_sf_atoms), _ptr(x_scale), _ptr(pw.codes),
                                          _ptr(pw.sf_atoms), _ptr(pw.tensor_scale), _ptr(r), M, pw.N,
                                          pw.K, pw.fmt, _ptr(out), ydt, token_tile,
                                          _stream(x_codes.device)), "dq_gemm_w4a4_fp4_tiled")
    return out


def linear_w4a4_fp4(x: torch.Tensor, a: Optional[torch.Tensor], pw: PackedFp4Weight,
                    r: Optional[torch.Tensor] = None, out_dtype=torch.float32) -> torch.Tensor:
    """Quantise activations (per-token second-level scale for NVFP4) and run the FP4 GEMM."""
    codes, sf_atoms, row_scale = quant_fp4(x, pw.fmt, a, None, atoms=True)
    return gemm_w4a4_fp4(codes, sf_atoms, row_scale, pw, r, out_dtype)


def mma_peak(kind: int, iters: int = 4096, device=None) -> float:
    """Tensor-pipe ceiling probe (dq_mma_peak_probe): tera-operations per second of a pure
    tcgen05.mma issue loop on every SM.  kind 0 = int8, 1 = MXFP4, 2 = NVFP4."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    _lib.ensure_init(idx)
    lib = _lib.load()
    n_ops = ctypes.c_double(0.0)
    stream = _stream(dev)
    _lib.check(lib.dq_mma_peak_probe(kind, 64, None, stream), "dq_mma_peak_probe")  # warm-up
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    _lib.check(lib.dq_mma_peak_probe(kind, iters, ctypes.byref(n_ops), stream), "dq_mma_peak_probe")
    e1.record()
    torch.cuda.synchronize(dev)
    return n_ops.value / (e0.elapsed_time(e1) * 1e-3) / 1e12


def rope_kv_append(qkv: torch.Tensor, cos_tab: torch.Tensor, sin_tab: torch.Tensor, pos, hq: int, hkv: int,
                   k_cache: torch.Tensor, v_cache: torch.Tensor, tokens_per_seq: int = 1) -> torch.Tensor:
    """RoPE on the query and key heads of qkv [B * S, (hq + 2 hkv) * d] (bf16, S = tokens_per_seq),
    key / value heads written to the caches [B, hkv, max_len, d] at positions pos .. pos + S - 1.
    pos: an int64 device tensor (read by the kernel, so the call can sit in a captured graph) or a
    Python int.  Returns the rotated queries as [B, hq, S, d] (a view of [B, S, hq, d])."""
    lib = _prep(qkv)
    S = int(tokens_per_seq)
    if S < 1 or qkv.shape[0] % S:
        raise ValueError("qkv rows must be a multiple of tokens_per_seq")
    B = qkv.shape[0] // S
    hd = k_cache.shape[-1]
    max_len = k_cache.shape[2]
    if qkv.dtype != torch.bfloat16 or qkv.stride(-1) != 1 or not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("rope_kv_append expects bf16 qkv rows and contiguous caches")
    if cos_tab.shape[0] < max_len or cos_tab.shape[1] != hd or not cos_tab.is_contiguous() or not sin_tab.is_contiguous():
        raise ValueError("cos / sin tables must be contiguous [>= max_len, head_dim]")
    q = torch.empty(B, S, hq, hd, dtype=torch.bfloat16, device=qkv.device)
    if isinstance(pos, torch.Tensor):
        if pos.dtype != torch.int64 or pos.device != qkv.device:
            raise ValueError("pos must be an int64 tensor on the device of qkv")
        pos_dev, pos_host = _ptr(pos), 0
    else:
        pos_dev, pos_host = None, int(pos)
    _lib.check(lib.dq_rope_kv_append(_ptr(qkv), qkv.stride(0), _ptr(cos_tab), _ptr(sin_tab), pos_dev, pos_host, B, S,
                                     hq, hkv, hd, max_len, _ptr(q), _ptr(k_cache), _ptr(v_cache),
                                     _stream(qkv.device)),
               "dq_rope_kv_append")
    return q.transpose(1, 2)
