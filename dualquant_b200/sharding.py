"""Column-parallel sharding of a single linear over the ranks of one node.

Rank p owns a contiguous range of output rows (whole 128-row weight tiles, so its slice of the
packed weight is one contiguous byte range); activations are replicated; outputs stay sharded.
There is no data-path collective: the only communication is the timing reduction of a benchmark.

Also the token bookkeeping of the decoder's token-sharded prompt pass (rank p owns the residual
stream of tokens [p * T / world, (p + 1) * T / world) of the flattened [batch, seq] prompt)."""
from __future__ import annotations

TILE = 128


def shard_rows(N: int, world: int, rank: int):
    """[start, end) of the output rows rank `rank` owns.  Tiles are dealt out as evenly as possible;
    the ranges of all ranks partition [0, N)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} / world {world}")
    tiles = (N + TILE - 1) // TILE
    base, extra = divmod(tiles, world)
    t0 = rank * base + min(rank, extra)
    t1 = t0 + base + (1 if rank < extra else 0)
    return min(t0 * TILE, N), min(t1 * TILE, N)


def token_shard(tokens: int, world: int, rank: int):
    """[start, end) of the flattened prompt tokens whose residual stream rank `rank` owns."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} / world {world}")
    if tokens % world:
        raise ValueError(f"{tokens} tokens do not divide over {world} ranks")
    tq = tokens // world
    return rank * tq, (rank + 1) * tq


def last_token_rows(batch: int, seq: int, world: int, rank: int):
    """The sequences whose last position this rank owns: [(sequence index, row in the rank's slice)]."""
    lo, hi = token_shard(batch * seq, world, rank)
    return [(b, b * seq + seq - 1 - lo) for b in range(batch) if lo <= b * seq + seq - 1 < hi]


def peer_exchange_fits(tokens: int, world: int, hidden: int, min_tokens: int = 512) -> bool:
    """Whether the prompt pass can run its exchange over peer memory: whole 256-token output tiles per
    owner, whole 128-row tiles of the hidden size, and enough tokens for the FP8-path GEMM."""
    return tokens % world == 0 and (tokens // world) % 256 == 0 and hidden % 128 == 0 and tokens >= min_tokens


def max_over_ranks(value: float, device=None) -> float:
    """MAX all-reduce of a scalar over the default process group (identity without one)."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
