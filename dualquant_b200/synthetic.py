"""Seeded synthetic operands with the shapes and value distributions of the benchmark
configurations: X ~ N(0,1) in bf16 with 1% outlier channels x20, W ~ N(0, 0.02) in bf16,
row / column scales log-normal(0, 0.3) rounded to fp16.  Generated on the CPU from an explicit
torch.Generator so that the same tensors can be fed to the library and to a checker."""
from __future__ import annotations

import torch

# (name, K, N) of every linear of one Llama-3.1-8B-architecture layer
LLAMA31_8B_LINEARS = (
    ("qkv", 4096, 6144),
    ("o", 4096, 4096),
    ("gate_up", 4096, 28672),
    ("down", 14336, 4096),
)
# Qwen2.5-7B-architecture linears (block-scaled FP4 configuration)
QWEN25_7B_LINEARS = (
    ("qkv", 3584, 4608),
    ("o", 3584, 3584),
    ("gate_up", 3584, 37888),
    ("down", 18944, 3584),
)
DECODE_M = (1, 8, 16, 32, 64, 128)


def make_x(M: int, K: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    outliers = torch.randperm(K, generator=g)[: K // 100]
    x[:, outliers] *= 20
    return x.to(torch.bfloat16)


def make_w(N: int, K: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 1)
    return (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)


def make_scales(N: int, K: int, seed: int = 0):
    """(r[N], c[K]) log-normal(0, 0.3), fp16-rounded, returned as fp32.  The vector multiplied
    into the activations is a = 1/c, computed in fp32 from the fp16 value of c."""
    g = torch.Generator().manual_seed(seed + 2)
    r = torch.exp(torch.randn(N, generator=g) * 0.3).to(torch.float16).to(torch.float32)
    c = torch.exp(torch.randn(K, generator=g) * 0.3).to(torch.float16).to(torch.float32)
    return r, c


def int4_gemm_bytes(M: int, N: int, K: int, group: int = 128) -> int:
    """Algorithmic bytes of one dual-scale int4 linear: packed weights + fp16 group scales +
    r + c (fp16) + bf16 activations in + fp32 output."""
    return N * K // 2 + N * (K // group) * 2 + 2 * N + 2 * K + 2 * M * K + 4 * M * N
