"""PermLinear: drop-in for the reference's runtime wrapper (activations/perm_linear.py:41-141,
activations/__init__.py:16-27) that runs the real W4A4 path on sm_100a.

Same constructor, attributes and methods as the reference module.  Where the reference
fake-quantises (quantise, de-quantise to bf16, bf16 F.linear against a fake-quant weight), this
module packs the wrapped layer's weight to int4 once and calls the library: fused activation
scale / online Hadamard / per-token int4 quantiser, then the int4 x int4 GEMM with exact int32
group sums and an fp32 epilogue.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _lib, ops
from .quarot import full_hadamard_scale, partial_hadamard_scale

GROUP = 128


class PermLinear(nn.Module):
    def __init__(self, layer: nn.Linear, act_fmt, quantize_bmm_input: bool = False):
        super().__init__()
        self.layer = layer
        self.dtype = layer.weight.dtype
        self.act_fmt = act_fmt  # FormatSpec
        self.quantize_bmm_input = quantize_bmm_input
        self.register_buffer("act_scale", None)

        # QuaRot online-Hadamard state, set by install_online_hadamards
        self.online_full_had = False
        self.online_partial_had = False
        self.had_K = None
        self.K = 1
        self.had_dim = 0
        self.fp32_had = False

        # False: the activation cast is skipped (the online Hadamard still runs)
        self.act_quant_enabled = True

        # packed weight artefact, built on first use (or by pack())
        self._packed: Optional[ops.PackedInt4Weight] = None
        self._packed_fp4: Optional[ops.PackedFp4Weight] = None
        self._hadamard_cache = None
        self._scratch: Optional[torch.Tensor] = None
        # None = not examined yet; False = the weight is not on the W4 grid of the activation
        # format, the layer keeps the reference's fake-quant formulation
        self._weight_on_grid: Optional[bool] = None
        self._weight_on_grid_fp4: Optional[bool] = None

    # ------------------------------------------------------------------ reference surface
    def set_act_scale(self, act_scale):
        if act_scale is not None:
            act_scale = act_scale.detach().clone().to(torch.float32)
        self.act_scale = act_scale

    def set_act_quant_enabled(self, enabled: bool) -> None:
        self.act_quant_enabled = bool(enabled)

    # ------------------------------------------------------------------ weight packing
    def pack(self, codes: Optional[torch.Tensor] = None, sw: Optional[torch.Tensor] = None,
             force: bool = False) -> bool:
        """Builds the int4 artefact.  Without arguments the wrapped layer's (fake-quant) weight is
        re-quantised per group of 128 along K, which is how the reference's real-kernel scripts
        recover codes and scales from `mat_q` (validate_real_kernel.py:95-98 via
        pack_int4_weights).  `codes` (int8 [N,K]) and `sw` (fp16 [N,K/128]) may be given directly.

        The reference's PermLinear never touches the weight (activations/perm_linear.py:136-141), so
        the real int4 GEMM may stand in for `F.linear(x_q, W)` only when W already lies on the int4
        group-of-128 grid.  After re-quantising, codes * scale must reproduce the stored weight to
        within the rounding of its storage type (1/128 of the group maximum); otherwise the weight is
        not W4-g128 (a 16-bit weight, per-row or GPTQ scales off this grid, another format) and the
        layer keeps the reference's formulation - fake-quantised activations into the wrapped
        layer's own F.linear.  `force=True` packs regardless (an explicit opt-in to quantising the
        weight here).  Returns True when the int4 artefact is in use."""
        w = self.layer.weight
        if not w.is_cuda:
            raise RuntimeError("PermLinear.pack needs the layer on a CUDA device (no CPU path)")
        if codes is None:
            w16 = w.detach().to(torch.bfloat16)
            codes, sw = ops.quant_w_int4(w16)
            if not force and not _reproduces(codes, sw, w.detach(), GROUP):
                self._packed = None
                self._weight_on_grid = False
                return False
        self._packed = ops.pack_w_int4(codes.to(w.device), sw.to(w.device))
        self._weight_on_grid = True
        return True

    def pack_fp4(self, fmt: int, force: bool = False) -> bool:
        """FP4 counterpart of pack(): the weight is packed in the activation format only when it
        already lies on that format's grid (its cast reproduces it), or with force=True."""
        w = self.layer.weight.detach()
        if not w.is_cuda:
            raise RuntimeError("PermLinear.pack_fp4 needs the layer on a CUDA device (no CPU path)")
        if not force:
            cast = self.act_fmt.cast(w.float())
            blk = 32 if fmt == _lib.FP4_MXFP4 else 16
            wb = w.float().reshape(w.shape[0], -1, blk)
            tol = wb.abs().amax(-1, keepdim=True) * (1.0 / 128.0)
            if not bool(((cast.reshape(wb.shape) - wb).abs() <= tol).all()):
                self._packed_fp4 = None
                self._weight_on_grid_fp4 = False
                return False
        self._packed_fp4 = ops.pack_w_fp4(w, fmt)
        self._weight_on_grid_fp4 = True
        return True

    def _hadamard(self, device) -> Optional[ops.Hadamard]:
        if not (self.online_full_had or self.online_partial_had):
            return None
        if self._hadamard_cache is not None and self._hadamard_cache[0] == device:
            return self._hadamard_cache[1]
        K = self.layer.in_features
        if self.online_full_had:
            mat = None if self.had_K is None else self.had_K.to(device=device, dtype=torch.float32).contiguous()
            had = ops.Hadamard(_lib.HAD_FULL, int(self.K), 0, full_hadamard_scale(K), mat)
        else:
            if self.K != 1:
                raise NotImplementedError("partial online Hadamard with a non-power-of-two head count")
            had = ops.Hadamard(_lib.HAD_PARTIAL, 1, int(self.had_dim),
                               partial_hadamard_scale(K // int(self.had_dim)), None)
        self._hadamard_cache = (device, had)
        return had

    def _fp4_fmt(self):
        name = getattr(self.act_fmt, "name", None)
        if not self.act_quant_enabled or name not in ("mxfp4", "nvfp4"):
            return None
        if self.online_full_had or self.online_partial_had or self.layer.in_features % 256 != 0:
            return None
        return _lib.FP4_MXFP4 if name == "mxfp4" else _lib.FP4_NVFP4

    def _bf16_arith(self, x2: torch.Tensor) -> bool:
        """The reference upcasts to fp32 only when an activation scale or an online Hadamard is
        configured; otherwise a bf16 input is quantised in bf16 arithmetic (perm_linear.py:109-133)."""
        return (x2.dtype == torch.bfloat16 and self.act_scale is None
                and not (self.online_full_had or self.online_partial_had))

    def _a16w4_ready(self) -> bool:
        """True when the layer can run 16-bit activations against its packed int4 weight: no online
        Hadamard, K a multiple of the group size, and the weight on the int4 grid (packs on demand)."""
        if self.online_full_had or self.online_partial_had or self.layer.in_features % GROUP != 0:
            return False
        if not self.layer.weight.is_cuda:
            return False
        if self._packed is None and self._weight_on_grid is None:
            self.pack()
        return self._packed is not None

    def _int4_path(self) -> bool:
        return (self.act_quant_enabled and getattr(self.act_fmt, "name", None) == "rtn_int4"
                and self.act_fmt.block_size == -1 and self.layer.in_features % GROUP == 0)

    # ------------------------------------------------------------------ forward
    def _quantise_act(self, x):
        """The reference's activation path as a de-quantised tensor (perm_linear.py:108-134);
        used when the int4 GEMM does not apply (act quant disabled, other formats)."""
        x2 = x.reshape(-1, x.shape[-1])
        had = self._hadamard(x.device)
        if self.act_quant_enabled:
            if getattr(self.act_fmt, "name", None) == "rtn_int4" and self.act_fmt.block_size == -1:
                xin = x2 if x2.dtype in (torch.bfloat16, torch.float32) else x2.float()
                out = ops.fakequant_act_int4(xin.contiguous(), self.act_scale, had, scale_fp16=False,
                                             bf16_arith=self._bf16_arith(xin))
            else:
                x32 = x2.float()
                if self.act_scale is not None:
                    x32 = x32 * self.act_scale
                if had is not None:
                    x32 = ops.hadamard_f32(x32, had)
                out = self.act_fmt.cast(x32)
        else:
            x32 = x2.float()
            if self.act_scale is not None:
                x32 = x32 * self.act_scale
            out = ops.hadamard_f32(x32, had) if had is not None else x32
        return out.to(self.dtype).reshape(x.shape)

    def forward(self, x):
        if not x.is_cuda:
            raise RuntimeError("dualquant_b200.PermLinear runs on CUDA (sm_100a) tensors only")
        use_int4 = self._int4_path()
        if use_int4 and self._packed is None and self._weight_on_grid is None:
            self.pack()
        fmt4 = None if use_int4 else self._fp4_fmt()
        if fmt4 is not None and (self._packed_fp4 is None or self._packed_fp4.fmt != fmt4) \
                and self._weight_on_grid_fp4 is None:
            self.pack_fp4(fmt4)
        if use_int4 and self._packed is not None:
            pw = self._packed
            x2 = x.reshape(-1, x.shape[-1])
            M = x2.shape[0]
            need = ops.linear_scratch_bytes(M, pw.N, pw.K)
            if self._scratch is None or self._scratch.numel() < need or self._scratch.device != x.device:
                self._scratch = torch.empty(max(need, 256), dtype=torch.uint8, device=x.device)
            out_dtype = self.dtype if self.dtype in (torch.bfloat16, torch.float32) else torch.float32
            if x2.dtype == torch.bfloat16:
                # without an activation scale and a Hadamard the reference quantises in the input
                # dtype, i.e. in bf16 arithmetic (perm_linear.py:109-133); same here
                out = ops.linear_w4a4_int4(x2, self.act_scale, self._hadamard(x.device), pw, None,
                                           out_dtype=out_dtype, scale_fp16=False, scratch=self._scratch,
                                           bf16_arith=self._bf16_arith(x2))
            else:
                # the reference upcasts to fp32 before scaling and quantising (perm_linear.py:119-125):
                # fp32 / fp16 inputs go through the fp32 quantiser, not through a bf16 rounding
                codes, sx = ops.quant_act_int4(x2.float(), self.act_scale, self._hadamard(x.device),
                                               scale_fp16=False)
                out = ops.gemm_w4a4_int4(codes, sx, pw, None, out_dtype=out_dtype)
            out = out.to(self.dtype)
            if self.layer.bias is not None:
                out = out + self.layer.bias
            out = out.reshape(x.shape[:-1] + (pw.N,))
        elif fmt4 is not None and self._packed_fp4 is not None and self._packed_fp4.fmt == fmt4:
            # block-scaled FP4 activations against the weight packed in the same format
            x2 = x.reshape(-1, x.shape[-1])
            if x2.dtype not in (torch.bfloat16, torch.float32):
                x2 = x2.float()
            out_dtype = self.dtype if self.dtype in (torch.bfloat16, torch.float32) else torch.float32
            out = ops.linear_w4a4_fp4(x2, self.act_scale, self._packed_fp4, None, out_dtype).to(self.dtype)
            if self.layer.bias is not None:
                out = out + self.layer.bias
            out = out.reshape(x.shape[:-1] + (self._packed_fp4.N,))
        elif (not self.act_quant_enabled and self._a16w4_ready()
              and x.dtype == torch.bfloat16 and self.dtype == torch.bfloat16):
            # activation cast switched off on a W4 layer: bf16(x * act_scale) against the packed int4
            # weight on the bf16 tensor cores (the reference multiplies by its 16-bit fake-quant copy)
            pw = self._packed
            x2 = x.reshape(-1, x.shape[-1])
            out = ops.linear_a16w4(x2, self.act_scale, pw, None, out_dtype=torch.bfloat16)
            if self.layer.bias is not None:
                out = out + self.layer.bias
            out = out.reshape(x.shape[:-1] + (pw.N,))
        else:
            out = self.layer(self._quantise_act(x))
        if self.quantize_bmm_input:
            if (out.dtype == torch.bfloat16 and getattr(self.act_fmt, "name", None) == "rtn_int4"
                    and self.act_fmt.block_size == -1 and out.shape[-1] % 8 == 0):
                # one pass, bf16 in and out: same values as cast(out.float()).to(bf16)
                out = ops.fakequant_act_int4_bf16(out.reshape(-1, out.shape[-1])).reshape(out.shape)
            else:
                out = self.act_fmt.cast(out.to(torch.float32)).to(self.dtype)
        return out


def _reproduces(codes: torch.Tensor, sw: torch.Tensor, w: torch.Tensor, group: int) -> bool:
    """True when codes * group scale gives back `w` up to the rounding of w's storage type."""
    N, K = codes.shape
    deq = codes.float().reshape(N, K // group, group) * sw.float().unsqueeze(-1)
    wg = w.float().reshape(N, K // group, group)
    tol = wg.abs().amax(-1, keepdim=True) * (1.0 / 128.0)
    return bool(((deq - wg).abs() <= tol).all())


def install_perm_linear(parent: nn.Module, attr_name: str, act_fmt, col_scales=None,
                        quantize_bmm_input: bool = False) -> PermLinear:
    """Wraps parent.<attr_name> (an nn.Linear) with a PermLinear in place and seeds its
    activation scale (activations/__init__.py:16-27)."""
    layer = getattr(parent, attr_name)
    perm = PermLinear(layer, act_fmt=act_fmt, quantize_bmm_input=quantize_bmm_input)
    perm.set_act_scale(col_scales)
    setattr(parent, attr_name, perm)
    return perm


__all__ = ["PermLinear", "install_perm_linear"]
