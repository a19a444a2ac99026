"""FormatSpec registry: drop-in for the reference's `formats` package
(formats/base.py:33-39, formats/__init__.py:29-44) restricted to the formats on the W4A4 hot
path.  `cast` runs on the GPU through the C ABI and returns the de-quantised tensor, exactly what
the reference's fake-quant casts return; CPU tensors are rejected (there is no CPU path)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from . import ops


@dataclass
class FormatSpec:
    """Same fields as the reference dataclass (formats/base.py:33-39)."""

    name: str
    block_size: int
    max_val: float
    cast: Callable[[torch.Tensor], torch.Tensor]
    cast_element_only: Callable[[torch.Tensor], torch.Tensor]


def _rtn_int4_cast(W: torch.Tensor, block_size: int) -> torch.Tensor:
    """formats/rtn_int.py:43-69 (`_rtn_cast`, qmax=7, qmin=-8): one absmax/7 scale per row per
    block (1 for an all-zero block), round-half-even, clamp, times the scale.  block_size == -1
    means one block per row (per-token for activations)."""
    if not W.is_cuda:
        raise RuntimeError("dualquant_b200 formats cast CUDA tensors only")
    orig_shape, orig_dtype = W.shape, W.dtype
    cols = orig_shape[-1]
    bs = cols if block_size == -1 else block_size
    if cols % bs != 0:
        raise ValueError(f"last dim {cols} is not a multiple of block_size {bs}")
    x = W.reshape(-1, bs)
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.to(torch.float32)
    # a bf16 tensor is cast in bf16 arithmetic, as torch evaluates the reference's expression on it
    out = ops.fakequant_act_int4(x.contiguous(), None, None, scale_fp16=False,
                                 bf16_arith=(x.dtype == torch.bfloat16))
    return out.reshape(orig_shape).to(orig_dtype)


def _rtn_cast_element_only(W: torch.Tensor, qmax: float, qmin: float) -> torch.Tensor:
    return W.clone().round_().clamp_(qmin, qmax)


def make_rtn_int4(block_size: int = 128, mse: bool = False) -> FormatSpec:
    if mse:
        raise NotImplementedError("MSE weight clipping is calibration-time and not part of this library")
    return FormatSpec(
        name="rtn_int4",
        block_size=block_size,
        max_val=7.0,
        cast=lambda W: _rtn_int4_cast(W, block_size),
        cast_element_only=lambda W: _rtn_cast_element_only(W, 7, -8),
    )


def _fp4_cast(W: torch.Tensor, fmt: int, block: int) -> torch.Tensor:
    if not W.is_cuda:
        raise RuntimeError("dualquant_b200 formats cast CUDA tensors only")
    from . import _lib

    orig_shape, orig_dtype = W.shape, W.dtype
    x = W.reshape(-1, orig_shape[-1])
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.to(torch.float32)
    ts = ops.nvfp4_tensor_scale(x) if fmt == _lib.FP4_NVFP4 else None
    return ops.fakequant_fp4(x, fmt, None, ts).reshape(orig_shape).to(orig_dtype)


def _float_to_fp4(W: torch.Tensor) -> torch.Tensor:
    """Element-only E2M1 rounding (legacy_vendor/torch_quant.py:326-356): the MXFP4 cast with the
    block exponent forced to 0 cannot be expressed through the block quantiser, so this is the
    same threshold table written with torch ops (calibration-time helper, not on the hot path)."""
    ax = W.abs()
    out = torch.zeros_like(ax)
    for thr, val, strict in ((0.25, 0.5, True), (0.75, 1.0, False), (1.25, 1.5, True), (1.75, 2.0, False),
                             (2.5, 3.0, True), (3.5, 4.0, False), (5.0, 6.0, True)):
        out = torch.where(ax > thr if strict else ax >= thr, torch.full_like(ax, val), out)
    return torch.where(W < 0, -out, out)


def make_mxfp4(block_size: int = 32) -> FormatSpec:
    """formats/mx.py:23-31.  Only the OCP block size 32 has a kernel."""
    from . import _lib

    if block_size != 32:
        raise NotImplementedError("mxfp4 is built for block_size 32 (the OCP MX block)")
    return FormatSpec(name="mxfp4", block_size=32, max_val=6.0,
                      cast=lambda W: _fp4_cast(W, _lib.FP4_MXFP4, 32),
                      cast_element_only=_float_to_fp4)


def make_nvfp4() -> FormatSpec:
    """formats/nvfp4.py:11-19: block 16, E4M3 block scale, per-tensor fp32 scale."""
    from . import _lib

    return FormatSpec(name="nvfp4", block_size=16, max_val=6.0,
                      cast=lambda W: _fp4_cast(W, _lib.FP4_NVFP4, 16),
                      cast_element_only=_float_to_fp4)


_FACTORIES = {"rtn_int4": make_rtn_int4, "mxfp4": make_mxfp4, "nvfp4": make_nvfp4}


def register_format(name: str, factory) -> None:
    _FACTORIES[name] = factory


def make_format(name: str, **fmt_cfg) -> FormatSpec:
    """formats/__init__.py:29-44.  Unknown names raise ValueError like the reference."""
    if name not in _FACTORIES:
        raise ValueError(f"unknown format {name!r}; expected one of {list(_FACTORIES)}")
    if name == "nvfp4":
        if fmt_cfg.get("block_size") not in (None, 16):
            raise ValueError(f"{name} block_size is fixed at 16 (got {fmt_cfg.get('block_size')})")
        return _FACTORIES[name]()
    if name != "rtn_int4":
        fmt_cfg.pop("mse", None)
    return _FACTORIES[name](**fmt_cfg)


__all__ = ["FormatSpec", "make_format", "register_format"]
