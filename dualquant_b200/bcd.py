"""DualQuant's offline weight step on the GPU: the alternating row / column scale search ("block
coordinate descent") of layer_wrapper_dualquant.py and the final block quantisation, for the int
formats of the W4A4 path.

Reference: wrap_dualquant_layer (layer_wrapper_dualquant.py:423-533) walks over the column blocks of
a weight one after the other on the CPU and runs, per block, dualquant_with_alpha_and_beta (:300-341),
dualquant_with_beta_only (:344-368) or dualquant_with_alpha_only (:371-394) followed by
_reconstruct_block_* (:403-420).  A block only ever sees its own rows x block_size columns, so all
blocks of a matrix are independent: here they are one batch - the weight is viewed as
[rows, blocks, block_size], the row scales alpha as [rows, blocks], the column scales beta as
[blocks, block_size] - and every step of the iteration is a handful of element-wise / reduction
launches over the whole matrix on its own device.  Same formulas, same initialisations, same scale
roundings; what differs from the reference's result is the order in which fp32 sums are formed
(and therefore, rarely, a code at a rounding boundary).

Covers quant_method "rtn_int4" / "rtn_int8" (the inner quantiser is the element-only integer cast,
layer_wrapper_dualquant.py:152-166; the stored weight is the per-row-of-block RTN block cast,
:193-200), scale formats "none", "e8m0", "e4m3" (:84-110) and num_splits = 1.  The FP4 block casts
of the reference go through the external blockfmt package and the e4m4 / e5m3 row-scale formats
through custom 9-bit helpers; neither is restated here.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

EPS = 1e-12                                            # layer_wrapper_dualquant.py:58
_E4M3_TINY = float(torch.finfo(torch.float8_e4m3fn).tiny)
_E4M3_MAX = float(torch.finfo(torch.float8_e4m3fn).max)

_QRANGE = {"rtn_int4": (-8.0, 7.0), "rtn_int8": (-128.0, 127.0)}


def _quantize_scale(scale: torch.Tensor, scale_format: str) -> torch.Tensor:
    """Row scale 1/alpha in its storage format (layer_wrapper_dualquant.py:84-147)."""
    if scale_format == "none":
        return scale
    if scale_format == "e4m3":
        return scale.clamp(min=_E4M3_TINY, max=_E4M3_MAX).to(torch.float8_e4m3fn).to(torch.float32)
    if scale_format == "e8m0":
        # nearest power of two: exponent + the leading mantissa bit, clamped to the E8M0 range
        bits = scale.contiguous().view(torch.int32)
        leading = (bits >> 22) & 1
        e = ((bits >> 23) & 0xFF) - 127 + leading
        e = e.clamp(min=-127, max=128)
        out = ((e + 127).to(torch.uint8).to(torch.int32) << 23).view(torch.float32)
        out = torch.where(torch.isnan(scale), torch.full_like(out, float("inf")), out)  # biased exponent 255
        return out.clamp(min=2.0 ** -127)
    raise NotImplementedError(f"row-scale format {scale_format!r} is not restated (supported: none, e8m0, e4m3)")


def _init_beta(W3: torch.Tensor, col_init: str) -> torch.Tensor:
    """Forward column scale per (block, column) (layer_wrapper_dualquant.py:246-259)."""
    if col_init == "l1_norm":
        stat = W3.abs().sum(dim=0).clamp(min=1e-8)
    elif col_init == "l2_norm":
        stat = torch.sqrt((W3 ** 2).sum(dim=0)).clamp(min=1e-8)
    elif col_init == "all_one":
        stat = torch.ones(W3.shape[1:], device=W3.device, dtype=W3.dtype)
    elif col_init == "max_abs":
        stat = W3.abs().amax(dim=0).clamp(min=1e-8)
    else:
        raise ValueError(f"unsupported col_init {col_init!r}")
    return 1.0 / stat


def _init_alpha(W3n: torch.Tensor, qmax: float, row_init: str) -> torch.Tensor:
    """Forward row scale per (row, block) on the column-normalised matrix (:262-277)."""
    if row_init == "max_abs":
        stat = W3n.abs().amax(dim=-1) / qmax
    elif row_init == "all_one":
        stat = torch.ones(W3n.shape[:2], device=W3n.device, dtype=W3n.dtype)
    else:
        raise ValueError(f"unsupported row_init {row_init!r}")
    return 1.0 / stat


def dualquant_scales(weight: torch.Tensor, *, block_size: int = 128, num_iter: int = 5,
                     scale_option: str = "row_column", row_init: str = "max_abs", col_init: str = "l1_norm",
                     scale_format: str = "none", quant_method: str = "rtn_int4"
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The scale search for every column block of `weight` [rows, cols] at once, on its device.
    Returns (alpha [rows, blocks], beta [blocks, block_size]), the forward scales: the quantiser
    sees alpha * W * beta."""
    if quant_method not in _QRANGE:
        raise NotImplementedError(f"quant_method {quant_method!r} is not restated (supported: {sorted(_QRANGE)})")
    qmin, qmax = _QRANGE[quant_method]
    R, C = weight.shape
    if C % block_size:
        raise ValueError(f"n_cols ({C}) must be divisible by block_size ({block_size})")
    W3 = weight.detach().to(torch.float32).reshape(R, C // block_size, block_size)
    if scale_option not in ("row_column", "only_column", "only_row"):
        raise ValueError(f"unknown scale_option {scale_option!r}")
    with torch.no_grad():
        ones_a = torch.ones(R, C // block_size, device=W3.device, dtype=torch.float32)
        ones_b = torch.ones(C // block_size, block_size, device=W3.device, dtype=torch.float32)
        if scale_option == "only_row":
            beta = ones_b
            alpha = _init_alpha(W3, qmax, row_init)
        else:
            beta = _init_beta(W3, col_init)
            alpha = _init_alpha(W3 * beta.unsqueeze(0), qmax, row_init) if scale_option == "row_column" else ones_a
        alpha_inv, beta_inv = 1.0 / alpha, 1.0 / beta

        def inner(a, b):  # element-only integer cast of the scaled matrix
            return (a.unsqueeze(-1) * W3 * b.unsqueeze(0)).round_().clamp_(qmin, qmax)

        for _ in range(num_iter):
            if scale_option != "only_column":      # least-squares row scale for the current codes
                M = inner(alpha, beta)
                Mb = M * beta_inv.unsqueeze(0)
                denom = (Mb ** 2).sum(dim=-1) + EPS
                alpha_inv = _quantize_scale((W3 * Mb).sum(dim=-1) / denom, scale_format)
                alpha = 1.0 / alpha_inv
            if scale_option != "only_row":         # least-squares column scale
                M = inner(alpha, beta)
                Ma = M * alpha_inv.unsqueeze(-1)
                denom = (Ma ** 2).sum(dim=0) + EPS
                beta_inv = (W3 * Ma).sum(dim=0) / denom
                beta = 1.0 / beta_inv
    return alpha, beta


def dualquant_weight(weight: torch.Tensor, *, block_size: int = 128, num_iter: int = 5,
                     scale_option: str = "row_column", row_init: str = "max_abs", col_init: str = "l1_norm",
                     scale_format: str = "none", quant_method: str = "rtn_int4"
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """What wrap_dualquant_layer(..., act_quant_flag=True) leaves behind: (mat_q, column_scales).
    mat_q [rows, cols] fp32 is the stored weight - (1 / alpha) * BlockRTN(alpha * W * beta), one RTN
    scale per (row, block) - and column_scales [cols] = 1 / beta is the vector the activations are
    divided by at run time (W ~ mat_q * column_scales).  `wrap.pack_from_dualquant(mat_q,
    column_scales)` turns the pair into the packed int4 artefact."""
    qmin, qmax = _QRANGE.get(quant_method, (None, None))
    alpha, beta = dualquant_scales(weight, block_size=block_size, num_iter=num_iter, scale_option=scale_option,
                                   row_init=row_init, col_init=col_init, scale_format=scale_format,
                                   quant_method=quant_method)
    R, C = weight.shape
    with torch.no_grad():
        W3 = weight.detach().to(torch.float32).reshape(R, C // block_size, block_size)
        scaled = alpha.unsqueeze(-1) * W3 * beta.unsqueeze(0)
        s = scaled.abs().amax(dim=-1, keepdim=True).clamp(min=1e-8) / qmax
        Wq = (scaled / s).round_().clamp_(qmin, qmax) * s
        if scale_option != "only_column":
            Wq = _quantize_scale(1.0 / alpha, scale_format).unsqueeze(-1) * Wq
        mat_q = Wq.reshape(R, C)
        column_scales = (1.0 / beta).reshape(C)
    return mat_q, column_scales


def wrap_dualquant_layer(layer: torch.nn.Linear, opt_config: dict, quant_method: str = "rtn_int4",
                         act_quant_flag: bool = True) -> Optional[torch.Tensor]:
    """Drop-in for the reference's wrap_dualquant_layer on the formats above (num_splits = 1):
    mutates layer.weight in place and returns the column scales when act_quant_flag is set,
    otherwise folds them back into the weight and returns None."""
    if opt_config.get("num_splits", 1) != 1:
        raise NotImplementedError("num_splits > 1 is not restated")
    if not opt_config.get("dualquant_to_element_tensor", True):
        raise NotImplementedError("the legacy block-format inner quantiser needs the external blockfmt package")
    mat_q, cs = dualquant_weight(layer.weight.data, block_size=opt_config["block_size"],
                                 num_iter=opt_config["num_iter"], scale_option=opt_config["scale_option"],
                                 row_init=opt_config.get("row_init", "max_abs"),
                                 col_init=opt_config.get("col_init", "l1_norm"),
                                 scale_format=opt_config["scale_format"], quant_method=quant_method)
    with torch.no_grad():
        if act_quant_flag:
            layer.weight.copy_(mat_q.to(layer.weight.dtype))
            return cs
        layer.weight.copy_((mat_q * cs.unsqueeze(0)).to(layer.weight.dtype))
    return None
