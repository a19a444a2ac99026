"""Decoder-stack harness on one GPU: cache consistency between prefill and decode."""
import pytest
import torch

from dualquant_b200 import decoder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_decode_after_prefill_matches_longer_prefill():
    cfg = decoder.DecoderConfig(hidden_size=512, num_attention_heads=8, num_key_value_heads=2,
                                head_dim=64, intermediate_size=28 * 64, num_hidden_layers=2,
                                vocab_size=1000)
    torch.manual_seed(0)
    model = decoder.Decoder(cfg, torch.device(DEV), tp=1, rank=0, seed=3)
    B, S = 3, 24
    model.alloc_cache(B, S + 4)
    ids = torch.randint(0, cfg.vocab_size, (B, S + 1), device=DEV)
    with torch.no_grad():
        ref = model.prefill(ids)                      # logits at position S from a full prefill
        model.prefill(ids[:, :S])                     # cache positions 0..S-1
        pos = torch.tensor([S], dtype=torch.int64, device=DEV)
        got = model.decode_step(ids[:, S], pos)       # token S through the cache path
    assert got.shape == (B, cfg.vocab_size)
    # same arithmetic per token (per-token quantisation), bf16 attention kernels may differ
    err = (got.float() - ref.float()).abs().max() / ref.float().abs().max()
    assert err < 5e-2, err
    assert torch.isfinite(got.float()).all()
