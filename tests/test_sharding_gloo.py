"""The N > 1 host logic on CPU: two gloo ranks shard a linear column-parallel, each evaluates its
slice with the oracle, and the gathered slices reproduce the unsharded result exactly."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dualquant_b200 import sharding, synthetic
from oracle import dq_oracle as O


def test_shard_rows_partition():
    for N in (4096, 6144, 28672, 3584, 4608, 200, 128, 1):
        for world in (1, 2, 4, 8):
            ranges = [sharding.shard_rows(N, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == N
            for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(s % 128 == 0 for s, e in ranges if e > s)
    with pytest.raises(ValueError):
        sharding.shard_rows(128, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 5, 640, 256
        x = synthetic.make_x(M, K, 0)
        w = synthetic.make_w(N, K, 0)
        r, c = synthetic.make_scales(N, K, 0)
        qx, sx, _ = O.quant_act_int4(x, 1.0 / c, None, True)
        n0, n1 = sharding.shard_rows(N, world, rank)
        qw, sw = O.quant_w_int4(w[n0:n1])
        y_local = O.epilogue(O.acc_int32(qx, qw), sw, r[n0:n1], sx)
        # 640 rows = 5 tiles -> slices of 384 and 256 columns: gather padded, then trim
        widths = [b - a for a, b in (sharding.shard_rows(N, world, p) for p in range(world))]
        padded = torch.zeros(M, max(widths))
        padded[:, : n1 - n0] = y_local
        parts = [torch.zeros_like(padded) for _ in range(world)]
        dist.all_gather(parts, padded)
        y = torch.cat([p[:, :wd] for p, wd in zip(parts, widths)], dim=1)
        qw_full, sw_full = O.quant_w_int4(w)
        y_ref = O.epilogue(O.acc_int32(qx, qw_full), sw_full, r, sx)
        assert torch.equal(y, y_ref)
        slowest = sharding.max_over_ranks(float(rank + 1))
        assert slowest == float(world)
        torch.save(torch.tensor([1]), os.path.join(out_dir, f"ok{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_column_parallel(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}.pt") for r in range(world))


def test_token_shard_bookkeeping():
    for B, S in ((8, 2048), (4, 160), (3, 8), (1, 16)):
        for world in (1, 2, 4, 8):
            if (B * S) % world:
                with pytest.raises(ValueError):
                    sharding.token_shard(B * S, world, 0)
                continue
            ranges = [sharding.token_shard(B * S, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == B * S
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            owners = [(b, r, row) for r in range(world) for b, row in sharding.last_token_rows(B, S, world, r)]
            assert sorted(b for b, _, _ in owners) == list(range(B))      # every sequence exactly once
            for b, r, row in owners:
                assert ranges[r][0] + row == b * S + S - 1
    assert sharding.peer_exchange_fits(16384, 8, 4096) and sharding.peer_exchange_fits(512, 2, 1024)
    assert not sharding.peer_exchange_fits(640, 2, 1024)      # 320 tokens per rank: not whole 256-token tiles
    assert not sharding.peer_exchange_fits(256, 1, 1024)      # too few tokens for the prefill GEMM
    assert not sharding.peer_exchange_fits(16384, 8, 4000)    # hidden size not in whole 128-row tiles


def _token_worker(rank, world, port, out_dir):
    """The data flow of the token-sharded prompt pass with the oracle's arithmetic: a row-parallel
    linear (each rank its K slice), partial outputs reduced onto the token owners, residual added on
    the slice, slices gathered again; against the all-reduce flow and the unsharded linear."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, S, H, K = 2, 4, 128, 512
        T = B * S
        x_res = synthetic.make_x(T, H, 1).float()                 # residual stream (replicated input)
        act = synthetic.make_x(T, K, 2)                           # input of the row-parallel linear
        w = synthetic.make_w(H, K, 3)
        k0, k1 = rank * K // world, (rank + 1) * K // world
        qx, sx, _ = O.quant_act_int4(act[:, k0:k1], None, None, False)   # per-shard token scales
        qw, sw = O.quant_w_int4(w[:, k0:k1])
        part = O.epilogue(O.acc_int32(qx, qw), sw, None, sx).to(torch.bfloat16)
        # all-reduce flow: every rank holds the whole stream
        full = part.float().clone()
        dist.all_reduce(full)
        x_allreduce = (x_res.to(torch.bfloat16).float() + full.to(torch.bfloat16).float()).to(torch.bfloat16)
        # token-sharded flow: sum in rank order onto the owner's slice, residual added there
        parts = [torch.zeros_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        lo, hi = sharding.token_shard(T, world, rank)
        acc = parts[0][lo:hi].float()
        for p in parts[1:]:
            acc = acc + p[lo:hi].float()
        x_slice = (x_res[lo:hi].to(torch.bfloat16).float() + acc.to(torch.bfloat16).float()).to(torch.bfloat16)
        slices = [torch.zeros_like(x_slice) for _ in range(world)]
        dist.all_gather(slices, x_slice)
        assert torch.equal(torch.cat(slices), x_allreduce)        # two ranks: two-term sums, same rounding
        # last position of every sequence, collected from its owner
        last = torch.zeros(B, H)
        for b, row in sharding.last_token_rows(B, S, world, rank):
            last[b] = x_slice[row].float()
        dist.all_reduce(last)
        assert torch.equal(last, x_allreduce.float()[[b * S + S - 1 for b in range(B)]])
        torch.save(torch.tensor([1]), os.path.join(out_dir, f"tok{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_token_sharded_flow(tmp_path):
    world = 2
    mp.spawn(_token_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"tok{r}.pt") for r in range(world))
