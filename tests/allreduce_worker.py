"""Child process of test_gpu_allreduce.py: one rank of a 2..8-rank run (torch.distributed.run).

Every rank holds the K slice of a row-parallel W4A4 int4 linear.  The fused all-reduce GEMM must
return, on every rank, the rank-ordered fp32 sum of the ranks' plain GEMM outputs - bit-exact,
because each rank's partial is computed by the same kernel arithmetic and summed in rank order.
NVLS is off and the kernel uses plain peer loads only.
"""
import os
import sys

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from dualquant_b200 import _lib, ops


def main():
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ctx = ops.AllReduceContext(dist.group.WORLD, dev, capacity_floats=16 * 8192)
    failures = []
    # (M, N, K per rank); N = 4096 with K = 7168 exercises split-K clusters plus the exchange
    cases = [(1, 4096, 2048), (8, 4096, 2048), (16, 4096, 7168), (5, 1024, 512), (16, 4100, 256), (3, 132, 128)]
    for it, (M, N, K) in enumerate(cases * 3):  # repeated: alternating buffer halves, growing epochs
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        codes = torch.randint(-8, 8, (M, K), generator=g, device=dev, dtype=torch.int8)
        sx = torch.rand(M, generator=g, device=dev) + 0.5
        wq = torch.randint(-8, 8, (N, K), generator=g, device=dev, dtype=torch.int8)
        sw = (torch.rand(N, K // 128, generator=g, device=dev) * 0.02 + 0.001).half()
        r = torch.rand(N, generator=g, device=dev) + 0.5
        pw = ops.pack_w_int4(wq, sw)
        part = ops.gemm_w4a4_int4(codes, sx, pw, r, out_dtype=torch.float32)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        want = torch.zeros_like(part)
        for p in parts:  # the kernel adds in rank order starting from zero
            want = want + p
        for dt in (torch.float32, torch.bfloat16):
            got = ops.gemm_w4a4_int4_ar(codes, sx, pw, r, ctx, out_dtype=dt)
            torch.cuda.synchronize(dev)
            if not torch.equal(got, want.to(dt)):
                failures.append((it, M, N, K, str(dt), float((got.float() - want).abs().max())))
            # with the residual connection added as the sum is stored (same tensor on every rank)
            gr = torch.Generator(device=dev).manual_seed(7 + it)
            res = torch.randn(M, N, generator=gr, device=dev).to(dt)
            got = ops.gemm_w4a4_int4_ar(codes, sx, pw, r, ctx, residual=res)
            torch.cuda.synchronize(dev)
            if not torch.equal(got, (want.to(dt).float() + res.float()).to(dt)):
                failures.append((it, M, N, K, str(dt), "residual"))
    status = _lib.device_status(local)
    # a CUDA graph holding several fused calls replays correctly
    M, N, K = 8, 4096, 2048
    g = torch.Generator(device=dev).manual_seed(999 + rank)
    codes = torch.randint(-8, 8, (M, K), generator=g, device=dev, dtype=torch.int8)
    sx = torch.rand(M, generator=g, device=dev) + 0.5
    wq = torch.randint(-8, 8, (N, K), generator=g, device=dev, dtype=torch.int8)
    sw = (torch.rand(N, K // 128, generator=g, device=dev) * 0.02 + 0.001).half()
    pw = ops.pack_w_int4(wq, sw)
    part = ops.gemm_w4a4_int4(codes, sx, pw, None, out_dtype=torch.float32)
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    want = sum(parts[1:], torch.zeros_like(part) + parts[0])
    outs = [torch.empty(M, N, device=dev) for _ in range(3)]
    torch.cuda.synchronize(dev)
    dist.barrier(device_ids=[local])
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for o in outs:
            ops.gemm_w4a4_int4_ar(codes, sx, pw, None, ctx, out=o)
    for rep in range(4):
        for o in outs:
            o.zero_()
        torch.cuda.synchronize(dev)
        dist.barrier(device_ids=[local])
        graph.replay()
        torch.cuda.synchronize(dev)
        for j, o in enumerate(outs):
            if not torch.equal(o, want):
                failures.append(("graph", rep, j, float((o - want).abs().max())))
    status = status or _lib.device_status(local)
    bad = torch.tensor([len(failures) + (1 if status else 0)], device=dev)
    dist.all_reduce(bad)
    if failures or status:
        print(f"rank {rank}: status={status} failures={failures[:5]}", flush=True)
    if rank == 0:
        print("ALLREDUCE_OK" if int(bad.item()) == 0 else "ALLREDUCE_FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(bad.item()) == 0 else 1)


if __name__ == "__main__":
    main()
