"""From DualQuant's offline outputs to the packed W4A4 artefact.

DualQuant's `method.wrap(layer, ...)` leaves the fake-quantised matrix `mat_q` in `layer.weight`
and returns the per-input-channel scales (`column_scales` = 1/beta) that the runtime multiplies
into the activations (layer_wrapper_dualquant.py:520-533); the real-kernel scripts cache the pair
on disk as `{"mat_q", "beta"}` (ablation/real_int4_kernel/wrap_cache.py:23-40) and recover int4
codes and group scales by re-quantising `mat_q` per group of 128 along K
(validate_real_kernel.py:95-98 through fused_dual_scale_kernel.py:156-189).  The helpers here do
the same on the GPU and hand the result to PermLinear.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from .activations import PermLinear, install_perm_linear


def pack_from_dualquant(mat_q: torch.Tensor,
                        column_scales: Optional[torch.Tensor] = None
                        ) -> Tuple[ops.PackedInt4Weight, Optional[torch.Tensor]]:
    """mat_q [N, K] (the fake-quant weight DualQuant wrote, on a CUDA device), column_scales [K]
    or None -> (packed int4 weight, fp32 activation scale a[K])."""
    if not mat_q.is_cuda:
        raise RuntimeError("pack_from_dualquant needs mat_q on a CUDA device (no CPU path)")
    if mat_q.dim() != 2 or mat_q.shape[1] % 128 != 0:
        raise ValueError(f"mat_q must be [N, K] with K % 128 == 0, got {tuple(mat_q.shape)}")
    codes, sw = ops.quant_w_int4(mat_q.detach().to(torch.bfloat16).contiguous())
    a = None
    if column_scales is not None:
        if column_scales.numel() != mat_q.shape[1]:
            raise ValueError("column_scales must have one entry per input channel")
        a = column_scales.detach().to(device=mat_q.device, dtype=torch.float32).contiguous()
    return ops.pack_w_int4(codes, sw), a


def load_wrap_cache(path: str) -> dict:
    """Reads one file of the reference's wrap cache: {"mat_q": [N, K], "beta": [K]} on CPU."""
    blob = torch.load(path, map_location="cpu")
    if not isinstance(blob, dict) or "mat_q" not in blob or "beta" not in blob:
        raise ValueError(f"{path}: not a wrap-cache file (expected keys 'mat_q' and 'beta')")
    return {"mat_q": blob["mat_q"], "beta": blob["beta"]}


def load_column_scales(path: str) -> Dict[str, torch.Tensor]:
    """Reads one of the scale files DualQuant's driver saves after calibration
    (methods/dualquant.py:59-66, shipped under scales_dualquant_rtn_int4/): a dict
    {"layer<idx>.<sublayer path>": column_scales [in_features] fp32} (keys built in main.py:201),
    the vectors PermLinear multiplies into the activations."""
    blob = torch.load(path, map_location="cpu")
    if not isinstance(blob, dict) or not blob:
        raise ValueError(f"{path}: not a DualQuant scale file (expected a non-empty dict)")
    out = {}
    for key, val in blob.items():
        if not (isinstance(key, str) and key.startswith("layer") and "." in key):
            raise ValueError(f"{path}: unexpected key {key!r} (expected 'layer<idx>.<sublayer path>')")
        if not (torch.is_tensor(val) and val.dim() == 1):
            raise ValueError(f"{path}: entry {key!r} is not a 1-D tensor")
        out[key] = val.detach().to(torch.float32)
    return out


def install_column_scales(model: nn.Module, scales: Dict[str, torch.Tensor], strict: bool = True) -> int:
    """Seeds the activation scale of every PermLinear named by a scale file: key
    "layer<idx>.<path>" addresses model.model.layers[idx].<path> (the walk of main.py:196-207).
    Returns the number of layers set; with strict=True a key that does not resolve to a PermLinear
    of matching width raises."""
    layers = model.model.layers
    n = 0
    for key, vec in scales.items():
        head, _, path = key.partition(".")
        mod = layers[int(head[len("layer"):])]
        try:
            for part in path.split("."):
                mod = getattr(mod, part)
        except AttributeError:
            if strict:
                raise KeyError(f"{key}: no such sublayer") from None
            continue
        if not isinstance(mod, PermLinear) or mod.layer.in_features != vec.numel():
            if strict:
                raise KeyError(f"{key}: not a PermLinear with {vec.numel()} input channels")
            continue
        mod.set_act_scale(vec.to(mod.layer.weight.device))
        n += 1
    return n


def install_from_wrap(parent: nn.Module, attr_name: str, mat_q: torch.Tensor, beta: torch.Tensor,
                      act_fmt, quantize_bmm_input: bool = False) -> PermLinear:
    """Copies mat_q into parent.<attr_name>.weight (as wrap_cached does), wraps the layer with a
    PermLinear whose activation scale is `beta` and packs the int4 artefact right away."""
    layer = getattr(parent, attr_name)
    with torch.no_grad():
        layer.weight.copy_(mat_q.to(device=layer.weight.device, dtype=layer.weight.dtype))
    perm = install_perm_linear(parent, attr_name, act_fmt, col_scales=beta.to(layer.weight.device),
                               quantize_bmm_input=quantize_bmm_input)
    if layer.weight.is_cuda and perm._int4_path():
        perm.pack()
    return perm


__all__ = ["pack_from_dualquant", "load_wrap_cache", "install_from_wrap", "load_column_scales",
           "install_column_scales"]
