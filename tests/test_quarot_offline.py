"""QuaRot offline folds (dualquant_b200/quarot_offline.py) on CPU: against the weights the reference's
own apply_r1 produced on a tiny random Llama (tests/golden/make_golden.py), and losslessness of the
rotations on a small fp64 model."""
import copy
import math
import types

import numpy as np
import torch

from dualquant_b200 import quarot_offline as QO


class _Norm(torch.nn.Module):
    def __init__(self, n, dtype):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(n, dtype=dtype))

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * self.weight


def _tiny_llama(H, heads, hd, inter, vocab, dtype):
    def lin(i, o):
        return torch.nn.Linear(i, o, bias=False, dtype=dtype)

    layer = torch.nn.Module()
    layer.self_attn, layer.mlp = torch.nn.Module(), torch.nn.Module()
    for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
        setattr(layer.self_attn, n, lin(H, H))
    layer.mlp.up_proj, layer.mlp.gate_proj, layer.mlp.down_proj = lin(H, inter), lin(H, inter), lin(inter, H)
    layer.input_layernorm, layer.post_attention_layernorm = _Norm(H, dtype), _Norm(H, dtype)
    model = torch.nn.Module()
    model.model = torch.nn.Module()
    model.model.layers = torch.nn.ModuleList([layer])
    model.model.embed_tokens = torch.nn.Embedding(vocab, H, dtype=dtype)
    model.model.norm = _Norm(H, dtype)
    model.lm_head = lin(H, vocab)
    model.config = types.SimpleNamespace(hidden_size=H, num_attention_heads=heads, head_dim=hd,
                                         tie_word_embeddings=False)
    return model


def _forward(model, ids, heads, hd, online):
    """Plain decoder forward; `online` applies the runtime halves of R2 (Hadamard across heads in
    front of o_proj) and R4 (full Hadamard in front of down_proj)."""
    x = model.model.embed_tokens(ids)
    H = x.shape[-1]
    for layer in model.model.layers:
        h = layer.input_layernorm(x)
        B, S, _ = h.shape
        q, k, v = (getattr(layer.self_attn, n)(h).view(B, S, heads, hd).transpose(1, 2) for n in ("q_proj", "k_proj", "v_proj"))
        mask = torch.full((S, S), float("-inf"), dtype=x.dtype).triu(1)
        a = (torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(hd) + mask, -1) @ v).transpose(1, 2).reshape(B, S, H)
        if online:
            a = QO._wht_last_axis(a.view(B, S, heads, hd).transpose(2, 3)).transpose(2, 3).reshape(B, S, H) / math.sqrt(heads)
        x = x + layer.self_attn.o_proj(a)
        h2 = layer.post_attention_layernorm(x)
        m = torch.nn.functional.silu(layer.mlp.gate_proj(h2)) * layer.mlp.up_proj(h2)
        if online:
            m = QO.hadamard_rows(m)
        x = x + layer.mlp.down_proj(m)
    return model.lm_head(model.model.norm(x))


def test_apply_r1_matches_the_reference_weights(golden):
    """Same tiny Llama (weights from the fixture), same +-1 diagonal (seed 78 on the global
    generator, as the reference draws it): every rotated weight against the reference's result."""
    model = _tiny_llama(64, 4, 16, 112, 48, torch.float32)
    sd = {k[len("r1_before__"):]: torch.from_numpy(v.copy()) for k, v in golden.items() if k.startswith("r1_before__")}
    model.model.embed_tokens.weight.data = sd["model.embed_tokens.weight"]
    model.lm_head.weight.data = sd["lm_head.weight"]
    model.model.norm.weight.data = sd["model.norm.weight"]
    layer = model.model.layers[0]
    layer.input_layernorm.weight.data = sd["model.layers.0.input_layernorm.weight"]
    layer.post_attention_layernorm.weight.data = sd["model.layers.0.post_attention_layernorm.weight"]
    for n in "qkvo":
        getattr(layer.self_attn, f"{n}_proj").weight.data = sd[f"model.layers.0.self_attn.{n}_proj.weight"]
    for n in ("gate", "up", "down"):
        getattr(layer.mlp, f"{n}_proj").weight.data = sd[f"model.layers.0.mlp.{n}_proj.weight"]
    torch.manual_seed(78)
    QO.apply_r1(model, rotate_mode="hadamard", apply_r2_r4=True)
    got = {"model.embed_tokens.weight": model.model.embed_tokens.weight, "lm_head.weight": model.lm_head.weight}
    for n in "qkvo":
        got[f"model.layers.0.self_attn.{n}_proj.weight"] = getattr(layer.self_attn, f"{n}_proj").weight
    for n in ("gate", "up", "down"):
        got[f"model.layers.0.mlp.{n}_proj.weight"] = getattr(layer.mlp, f"{n}_proj").weight
    for name, w in got.items():
        ref = torch.from_numpy(golden["r1_after__" + name])
        # fp64 products rounded to fp32; the Hadamard folds run in fp32 with the same butterfly order
        assert torch.allclose(w.data, ref, rtol=0, atol=2e-6 * ref.abs().max().item()), name
    assert torch.equal(model.model.norm.weight.data, torch.ones(64))


def test_rotations_are_lossless_in_fp64():
    torch.manual_seed(0)
    H, heads, hd, inter, vocab = 64, 4, 16, 112, 50
    model = _tiny_llama(H, heads, hd, inter, vocab, torch.float64)
    for p in model.parameters():
        if p.dim() == 1:
            p.data = torch.rand_like(p) + 0.5
    ids = torch.randint(0, vocab, (2, 7))
    ref = _forward(model, ids, heads, hd, False)
    for mode in ("hadamard", "random"):
        m1 = copy.deepcopy(model)
        Q = QO.apply_r1(m1, mode, apply_r2_r4=False, generator=torch.Generator().manual_seed(3))
        assert torch.allclose(Q @ Q.T, torch.eye(H, dtype=torch.float64), atol=1e-10)
        assert (_forward(m1, ids, heads, hd, False) - ref).abs().max() < 1e-10   # R1 alone: exact
        m2 = copy.deepcopy(model)
        QO.apply_r1(m2, mode, apply_r2_r4=True, generator=torch.Generator().manual_seed(3))
        # R2 / R4 cancel only together with their online halves (their offline folds run in fp32)
        assert (_forward(m2, ids, heads, hd, True) - ref).abs().max() < 1e-5
        assert (_forward(m2, ids, heads, hd, False) - ref).abs().max() > 1e-2


def test_hadamard_rows_is_orthonormal_for_every_decomposition():
    for n in (64, 112, 96, 160):  # 2^6, 28*4, 12*8, 20*8 -> get_hadK picks 40*4 for 160
        x = torch.eye(n, dtype=torch.float64)
        h = QO.hadamard_rows(x)
        assert torch.allclose(h @ h.T, torch.eye(n, dtype=torch.float64), atol=1e-12)
