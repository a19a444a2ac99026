"""Online-Hadamard installation: drop-in for quarot/online_had_install.py:21-62 and the parts
of quarot/vendor/hadamard_utils.py:5-55 it needs."""
from __future__ import annotations

import math

import torch


def _is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


def _legendre(a: int, q: int) -> int:
    a %= q
    if a == 0:
        return 0
    return 1 if pow(a, (q - 1) // 2, q) == 1 else -1


def _quadratic_character_matrix(q: int) -> torch.Tensor:
    """Q[i][j] = legendre(j - i) for a prime q (the Jacobsthal matrix of GF(q))."""
    chi = torch.tensor([_legendre(d, q) for d in range(q)], dtype=torch.float32)
    idx = (torch.arange(q).reshape(1, q) - torch.arange(q).reshape(q, 1)) % q
    return chi[idx]


def paley1_hadamard(q: int) -> torch.Tensor:
    """Paley type-I Hadamard matrix of order q + 1 for a prime q = 3 (mod 4), in the normalisation
    of the matrices the reference stores as literals for the orders 12, 20, 60, 108 and 140
    (quarot/vendor/hadamard_utils.py:57-275): first column +1, rest of the first row -1, core
    I + Q^T with Q[i][j] = legendre(j - i)."""
    n = q + 1
    H = torch.ones(n, n)
    H[0, 1:] = -1
    H[1:, 1:] = torch.eye(q) + _quadratic_character_matrix(q).T
    return H.float()


def paley2_hadamard(q: int) -> torch.Tensor:
    """Paley type-II Hadamard matrix of order 2(q+1) for a prime q = 1 (mod 4):
    [[S+I, S-I], [S-I, -S-I]] with S = [[0, 1^T], [1, Q]], Q[i][j] = legendre(j-i).
    q = 13 gives the 28x28 matrix the reference stores as a literal
    (quarot/vendor/hadamard_utils.py:277-391), q = 17 its 36x36 one."""
    n = q + 1
    S = torch.zeros(n, n)
    S[0, 1:] = 1
    S[1:, 0] = 1
    S[1:, 1:] = _quadratic_character_matrix(q)
    eye = torch.eye(n)
    return torch.cat([torch.cat([S + eye, S - eye], 1), torch.cat([S - eye, -S - eye], 1)], 0).float()


# Williamson sequences: first rows (1 = +1, 0 = -1) of the four symmetric circulant blocks A, B, C, D
# with A^2 + B^2 + C^2 + D^2 = 4m I, for the orders 4m = 52, 156, 172 (block sizes 13, 39, 43) - the
# "will" matrices of N. J. A. Sloane's library of Hadamard matrices that QuaRot ships as literals.
_WILLIAMSON = {
    52: ("1010011110010", "1000111111000", "1101001100101", "1000010010000"),
    156: ("111001010000010011000011001000001010011", "111100010011000010100101000011001000111",
          "111001101000101001000010010100010110011", "100011010100000111011011100000101011000"),
    172: ("1000110011110101110110011011101011110011000", "1101111110000101001101101100101000011111101",
          "1110101100101011110100001011110101001101011", "1100011110100100110000000011001001011110001"),
}


def williamson_hadamard(order: int) -> torch.Tensor:
    """Williamson array [[A, B, C, D], [-B, A, -D, C], [-C, D, A, -B], [-D, -C, B, A]] of four
    circulant blocks whose first rows are the sequences above."""
    m = order // 4

    def circulant(bits: str) -> torch.Tensor:
        row = torch.tensor([1.0 if b == "1" else -1.0 for b in bits])
        idx = (torch.arange(m).reshape(1, m) - torch.arange(m).reshape(m, 1)) % m
        return row[idx]

    A, B, C, D = (circulant(b) for b in _WILLIAMSON[order])
    return torch.cat([torch.cat([A, B, C, D], 1), torch.cat([-B, A, -D, C], 1),
                      torch.cat([-C, D, A, -B], 1), torch.cat([-D, -C, B, A], 1)], 0).float()


def hadamard_of_order(k: int) -> torch.Tensor:
    """The k x k +-1 matrix the reference's get_hadK returns for order k
    (quarot/vendor/hadamard_utils.py:5-55), generated instead of stored."""
    if k in (12, 20, 60, 108, 140):
        return paley1_hadamard(k - 1)
    if k in (28, 36):
        return paley2_hadamard(k // 2 - 1)
    if k == 40:  # Sylvester doubling of the order-20 Paley matrix
        h = paley1_hadamard(19)
        return torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    if k in _WILLIAMSON:
        return williamson_hadamard(k)
    raise ValueError(f"no Hadamard matrix of order {k} in the reference's table")


# orders the reference tries, in its order (hadamard_utils.py:5-55)
_REFERENCE_ORDERS = (172, 156, 140, 108, 60, 52, 36, 28, 40, 20, 12)


def get_hadK(n: int, transpose: bool = False):
    """(had_K, K) with n = K * 2^m: the first order of the reference's table that divides n (the
    reference asserts that the cofactor is a power of two), or (None, 1) for a power of two."""
    for k in _REFERENCE_ORDERS:
        if n % k == 0:
            assert _is_pow2(n // k)
            h = hadamard_of_order(k)
            return (h.T.contiguous() if transpose else h), k
    assert _is_pow2(n)
    return None, 1


def full_hadamard_scale(n: int) -> float:
    """The fp32 factor of matmul_hadU_cuda (hadamard_utils.py:97-99)."""
    return float((1.0 / torch.tensor(n).sqrt()).item())


def partial_hadamard_scale(num_heads: int) -> float:
    """perm_linear.py:96-98: 1/sqrt(H) as applied to an fp32 tensor."""
    return float(torch.tensor(1.0 / math.sqrt(num_heads), dtype=torch.float32).item())


def install_online_hadamards(model, fp32_had: bool = False, verbose: bool = False) -> None:
    """Sets the online-Hadamard attributes on every PermLinear wrapping a down_proj (full
    transform of size intermediate_size) or an o_proj (partial transform across heads), reading
    the sizes from model.config - same walk as quarot/online_had_install.py:30-58."""
    from .activations import PermLinear

    cfg = model.config
    intermediate_size = int(cfg.intermediate_size)
    num_heads = int(cfg.num_attention_heads)
    head_dim = int(getattr(cfg, "head_dim", None) or (int(cfg.hidden_size) // num_heads))
    n_full = n_partial = 0
    for name, mod in model.named_modules():
        if not isinstance(mod, PermLinear):
            continue
        if "down_proj" in name:
            mod.had_K, mod.K = get_hadK(intermediate_size)
            mod.online_full_had = True
            mod.fp32_had = fp32_had
            n_full += 1
        elif "o_proj" in name:
            mod.had_K, mod.K = get_hadK(num_heads)
            mod.online_partial_had = True
            mod.had_dim = head_dim
            mod.fp32_had = fp32_had
            n_partial += 1
        else:
            continue
        mod._hadamard_cache = None
    if verbose:
        print(f"[quarot] installed online Hadamards: {n_full} down_proj (full), {n_partial} o_proj (partial)")


__all__ = ["get_hadK", "hadamard_of_order", "install_online_hadamards", "paley1_hadamard", "paley2_hadamard",
           "williamson_hadamard"]
