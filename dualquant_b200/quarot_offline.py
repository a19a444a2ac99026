"""QuaRot offline folds for Llama-family models, on whatever device the model lives on (GPU for real
checkpoints): RMSNorm fusion and the R1 / R2 / R4 weight rotations whose online halves
`install_online_hadamards` switches on.  Calibration-time companion of the W4A4 path - plain torch
matmuls in fp64 (the reference does the same, on its `utils.DEV`), not a kernel of its own.

Mirrors quarot/llama_quarot.py:186-264 (`apply_r1`) and the vendored helpers it drives:
quarot/vendor/rotation_utils.py:10-25 (`fuse_ln_linear`), :93-112 (random orthogonal / randomised
Hadamard Q), :116-176 (`rotate_embeddings`, `rotate_attention_inputs/output`, `rotate_mlp_input/
output`), :207-227 (`rotate_head`, `rotate_ov_proj`) and quarot/vendor/hadamard_utils.py:58-90,
108-141 (`matmul_hadU`, `random_hadamard_matrix`, `apply_exact_had_to_linear`).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .quarot import _is_pow2, get_hadK


def _wht_last_axis(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised Walsh-Hadamard transform over the last axis (Sylvester order, stages
    h = 1, 2, 4, ...: (a, b) -> (a + b, a - b)), as quarot/__init__.py:39-64."""
    n = x.shape[-1]
    assert _is_pow2(n)
    out = x.clone()
    h = 1
    while h < n:
        y = out.reshape(*out.shape[:-1], n // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        out = torch.stack((a + b, a - b), dim=-2).reshape(*out.shape[:-1], n)
        h *= 2
    return out


def hadamard_rows(x: torch.Tensor) -> torch.Tensor:
    """x @ H_n / sqrt(n) along the last axis with H_n = had_K (x) Walsh-Hadamard, the transform of
    matmul_hadU_cuda (quarot/vendor/hadamard_utils.py:92-101): view(-1, K, n/K), WHT over the last
    axis times 1/sqrt(n), then had_K @ ."""
    n = x.shape[-1]
    had_k, k = get_hadK(n)
    scale = 1.0 / torch.tensor(n).sqrt().to(x.dtype)
    if k == 1:
        return _wht_last_axis(x) * scale
    v = _wht_last_axis(x.reshape(-1, k, n // k)) * scale
    return (had_k.to(device=x.device, dtype=x.dtype) @ v).reshape(x.shape)


def random_hadamard_matrix(size: int, device, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """H_size / sqrt(size) times a random +-1 diagonal, fp64 (hadamard_utils.py:85-90)."""
    d = torch.randint(0, 2, (size,), generator=generator).to(torch.float64) * 2 - 1
    return hadamard_rows(torch.diag(d)).to(device)


def random_orthogonal_matrix(size: int, device, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """QR of a Gaussian matrix with the sign convention of rotation_utils.py:93-104."""
    m = torch.randn(size, size, dtype=torch.float64, generator=generator).to(device)
    q, r = torch.linalg.qr(m)
    return q * torch.sign(torch.diag(r)).unsqueeze(0)


def get_orthogonal_matrix(size: int, mode: str, device, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    if mode == "random":
        return random_orthogonal_matrix(size, device, generator)
    if mode == "hadamard":
        return random_hadamard_matrix(size, device, generator)
    raise ValueError(f"Unknown mode {mode}")


def _right(linear: torch.nn.Linear, Q: torch.Tensor) -> None:
    """W <- W @ Q (rotation of the layer's inputs), fp64."""
    w = linear.weight.data
    linear.weight.data = torch.matmul(w.to(device=Q.device, dtype=torch.float64), Q).to(device=w.device, dtype=w.dtype)


def _left_t(linear: torch.nn.Linear, Q: torch.Tensor) -> None:
    """W <- Q^T @ W, b <- Q^T @ b (rotation of the layer's outputs), fp64."""
    w = linear.weight.data
    linear.weight.data = torch.matmul(Q.T, w.to(device=Q.device, dtype=torch.float64)).to(device=w.device, dtype=w.dtype)
    if linear.bias is not None:
        b = linear.bias.data
        linear.bias.data = torch.matmul(Q.T, b.to(device=Q.device, dtype=torch.float64)).to(device=b.device, dtype=b.dtype)


def fuse_ln_linear(norm: torch.nn.Module, linears) -> None:
    """Folds the norm's weight into the linears that read its output (rotation_utils.py:10-25)."""
    for lin in linears:
        dt = lin.weight.dtype
        w64 = lin.weight.data.double()
        lin.weight.data = (w64 * norm.weight.double().to(w64.device)).to(dt)
        if getattr(norm, "bias", None) is not None:
            if lin.bias is None:
                lin.bias = torch.nn.Parameter(torch.zeros(lin.out_features, dtype=torch.float64, device=w64.device))
            lin.bias.data = (lin.bias.data.double() + torch.matmul(w64, norm.bias.double().to(w64.device))).to(dt)


def fuse_rmsnorms(model) -> None:
    """RMSNorm weights folded into q/k/v, gate/up and lm_head; the norms are left with unit weight
    (the reference swaps in a weight-less RMSNorm module, llama_quarot.py:103-141,152-178)."""
    for layer in model.model.layers:
        fuse_ln_linear(layer.post_attention_layernorm, [layer.mlp.up_proj, layer.mlp.gate_proj])
        fuse_ln_linear(layer.input_layernorm, [layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj])
        for norm in (layer.post_attention_layernorm, layer.input_layernorm):
            norm.weight.data = torch.ones_like(norm.weight.data)
    fuse_ln_linear(model.model.norm, [model.lm_head])
    model.model.norm.weight.data = torch.ones_like(model.model.norm.weight.data)


def apply_exact_had_to_linear(linear: torch.nn.Linear, had_dim: int = -1, output: bool = False) -> None:
    """hadamard_utils.py:108-141 in fp32: had_dim = -1 transforms the whole input (output=False) or
    output (output=True) axis; had_dim = d with output=True transforms every block of d outputs."""
    w = linear.weight.data
    w32 = w.float()
    if had_dim == -1:
        w32 = hadamard_rows(w32.t().contiguous()).t() if output else hadamard_rows(w32)
    else:
        if not _is_pow2(had_dim):
            raise ValueError("Hadamard dimension must be a power of 2")
        if not output:
            raise NotImplementedError("per-block input transform (not used by the reference either)")
        wt = w32.t().contiguous()
        shape = wt.shape
        wt = _wht_last_axis(wt.reshape(-1, shape[-1] // had_dim, had_dim)) * (1.0 / math.sqrt(had_dim))
        w32 = wt.reshape(shape).t()
    linear.weight.data = w32.contiguous().to(dtype=w.dtype)


def _untie_lm_head(model) -> None:
    model.lm_head.weight = torch.nn.Parameter(model.lm_head.weight.data.clone())
    if hasattr(model, "config"):
        model.config.tie_word_embeddings = False


@torch.no_grad()
def apply_r1(model, rotate_mode: str = "random", apply_r2_r4: bool = True, verbose: bool = False,
             generator: Optional[torch.Generator] = None, Q: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In place: fuse RMSNorms, rotate the residual stream by Q (R1) and, with apply_r2_r4, fold the
    offline halves of R2 (per-head Hadamard on v_proj outputs, full Hadamard on o_proj inputs) and
    R4 (full Hadamard on down_proj inputs) - same order of operations as llama_quarot.py:186-264.
    Returns Q (fp64).  R1 alone is lossless; R2 / R4 are lossless together with the online halves
    that `install_online_hadamards` enables."""
    if getattr(model.config, "tie_word_embeddings", False):
        _untie_lm_head(model)
    fuse_rmsnorms(model)
    dev = model.lm_head.weight.device
    if Q is None:
        Q = get_orthogonal_matrix(int(model.config.hidden_size), rotate_mode, dev, generator)
    Q = Q.to(device=dev, dtype=torch.float64)
    _right(model.model.embed_tokens, Q)
    _right(model.lm_head, Q)
    cfg = model.config
    num_heads = int(cfg.num_attention_heads)
    head_dim = int(getattr(cfg, "head_dim", None) or (int(cfg.hidden_size) // num_heads))
    for idx, layer in enumerate(model.model.layers):
        for lin in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj):
            _right(lin, Q)
        _left_t(layer.self_attn.o_proj, Q)
        for lin in (layer.mlp.up_proj, layer.mlp.gate_proj):
            _right(lin, Q)
        _left_t(layer.mlp.down_proj, Q)
        if apply_r2_r4:
            apply_exact_had_to_linear(layer.mlp.down_proj, had_dim=-1, output=False)          # R4
            apply_exact_had_to_linear(layer.self_attn.v_proj, had_dim=head_dim, output=True)  # R2
            apply_exact_had_to_linear(layer.self_attn.o_proj, had_dim=-1, output=False)
        if verbose:
            print(f"[quarot] layer {idx} rotated")
    return Q


__all__ = ["apply_r1", "apply_exact_had_to_linear", "fuse_rmsnorms", "fuse_ln_linear", "get_orthogonal_matrix",
           "hadamard_rows", "random_hadamard_matrix", "random_orthogonal_matrix"]
