"""Child process of test_gpu_decoder_tp.py: one rank of a tensor-parallel decoder stack
(torch.distributed.run, one process per GPU, NCCL with NVLS off).

Three prompt paths of the same sharded model must agree: the residual stream all-reduced after every
row-parallel linear (norms and quantisers replicated); the residual stream sharded over tokens with
NCCL (reduce-scatter of the partial outputs, all-gather of the activation codes); and the same
sharding with the exchange in this library's kernels over peer memory.  A fourth run replaces NCCL's
reduce-scatter by an all-gather and an fp32 sum in rank order - the arithmetic of the peer-memory
path - and must equal that path bit for bit at any number of ranks (with more than two ranks the
collectives' own summation orders differ at bf16 rounding level, and a W4A4 stack amplifies that
through flipped int4 codes, so those runs are only checked for finite, correlated logits).  With two ranks a sum
has two terms, so both orders round alike and the logits, the caches and the first decode step
must be equal bit for bit; with more ranks they agree to bf16 rounding of the partial sums.
"""
import os
import sys

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from dualquant_b200 import _lib, decoder


def _ordered_reduce_scatter(out, inp, group=None):
    """reduce_scatter_tensor as the peer-memory path computes it: fp32, rank order, rounded once."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    parts = [torch.empty_like(inp) for _ in range(world)]
    dist.all_gather(parts, inp, group=group)
    tq = out.shape[0]
    acc = parts[0][rank * tq:(rank + 1) * tq].float()
    for p in parts[1:]:
        acc = acc + p[rank * tq:(rank + 1) * tq].float()
    out.copy_(acc.to(out.dtype))


def main():
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = decoder.DecoderConfig(hidden_size=1024, num_attention_heads=8, num_key_value_heads=world,
                                head_dim=128, intermediate_size=28 * 64 * world, num_hidden_layers=2,
                                vocab_size=1000)
    # the same sharded model three times: all-reduce pass, token-sharded pass over NCCL, token-sharded
    # pass over peer memory (GEMM epilogues push their tiles to the owners; device-side barriers)
    models = [decoder.Decoder(cfg, dev, tp=world, rank=rank, seed=5, group=dist.group.WORLD,
                              token_sharded_prefill=flag, prefill_exchange=how)
              for flag, how in ((False, "nccl"), (True, "nccl"), (True, "peer"), (True, "nccl"))]
    stock_reduce_scatter = dist.reduce_scatter_tensor
    failures = []
    # 640 tokens: E4M3 codes and the FP8-path GEMM; 66 tokens: int8 codes, small-batch kernels;
    # 3 x 7 tokens with three ranks or more does not divide: the sharded path must step aside
    # 256 and 512 tokens per rank are what the peer-memory exchange takes (whole 256-token tiles per
    # owner); the other shapes make it fall back to NCCL
    for B, S in ((4, 160), (world, 256), (2 * world, 256), (2, 33 * world // 2 if world % 2 == 0 else 33 * world),
                 (3, 7), (world, 256)):
        g = torch.Generator().manual_seed(B * 1000 + S)   # CPU generator: the same prompt on every rank
        ids = torch.randint(0, cfg.vocab_size, (B, S), generator=g).to(dev)
        dist.broadcast(ids, src=0)
        outs = []
        with torch.no_grad():
            for which, m in enumerate(models):
                m.alloc_cache(B, S + 4)
                dist.reduce_scatter_tensor = _ordered_reduce_scatter if which >= 2 else stock_reduce_scatter
                logits = m.prefill(ids)
                dist.reduce_scatter_tensor = stock_reduce_scatter
                tok = logits.argmax(dim=-1)
                pos = torch.tensor([S], dtype=torch.int64, device=dev)
                step = m.decode_step(tok, pos)
                torch.cuda.synchronize(dev)
                outs.append((logits.float(), step.float(), m.layers[-1].k_cache[:, :, :S].float()))
        # the peer-memory pass replayed from a CUDA graph (barrier epochs counted on the device)
        if models[2]._peer_exchange(B, S):
            with torch.no_grad():
                run = models[2].capture_prefill(ids)
                for _ in range(2):
                    logits_g = run().float()
                    torch.cuda.synchronize(dev)
                    if not hasattr(run, "graph") or not torch.equal(logits_g, outs[2][0]):
                        failures.append(("captured peer pass", B, S, float((logits_g - outs[2][0]).abs().max())))

        def diffs(a, b):
            return tuple(float((x - y).abs().max()) for x, y in zip(a, b))

        def same(a, b):
            return all(torch.equal(x, y) for x, y in zip(a, b))

        # the peer-memory pass against the run with its arithmetic spelled out in torch: always exact
        if not same(outs[2], outs[3]):
            failures.append(("peer vs ordered sum", B, S) + diffs(outs[2], outs[3]))
        for which in (1, 2):
            if world == 2 or (B * S) % world != 0:
                ok = same(outs[0], outs[which])
            else:
                l0, l1 = outs[0][0].flatten(), outs[which][0].flatten()
                ok = bool(torch.isfinite(l1).all()) and float(torch.corrcoef(torch.stack([l0, l1]))[0, 1]) > 0.8
            if not ok:
                failures.append((which, B, S) + diffs(outs[0], outs[which]))
    if len(models[2]._exchange) != 2:  # 256 and 512 tokens per rank went over peer memory
        failures.append(("peer exchange contexts", sorted(models[2]._exchange)))
    status = 0
    try:
        _lib.device_status(local)
    except RuntimeError as exc:
        status = 1
        print(f"rank {rank}: {exc}", flush=True)
    bad = torch.tensor([len(failures) + status], device=dev)
    dist.all_reduce(bad)
    if failures:
        print(f"rank {rank}: failures={failures}", flush=True)
    if rank == 0:
        print("DECODER_TP_OK" if int(bad.item()) == 0 else "DECODER_TP_FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(bad.item()) == 0 else 1)


if __name__ == "__main__":
    main()
