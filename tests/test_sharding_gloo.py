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
