"""Child process of test_gpu_decoder_tp.py: one rank of a tensor-parallel decoder stack
(torch.distributed.run, one process per GPU, NCCL with NVLS off).

Three prompt paths of the same sharded model must agree: the residual stream all-reduced after every
row-parallel linear (norms and quantisers replicated); the residual stream sharded over tokens with
NCCL (reduce-scatter of the partial outputs, all-gather of the activation codes); and the same
sharding with the exchange in this library's kernels over peer memory.  With two ranks a sum
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
              for flag, how in ((False, "nccl"), (True, "nccl"), (True, "peer"))]
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
            for m in models:
                m.alloc_cache(B, S + 4)
                logits = m.prefill(ids)
                tok = logits.argmax(dim=-1)
                pos = torch.tensor([S], dtype=torch.int64, device=dev)
                step = m.decode_step(tok, pos)
                torch.cuda.synchronize(dev)
                outs.append((logits.float(), step.float(), m.layers[-1].k_cache[:, :, :S].float()))
        l0, s0, k0 = outs[0]
        for which, (l1, s1, k1) in enumerate(outs[1:], start=1):
            if world == 2 or (B * S) % world != 0:
                same = torch.equal(l0, l1) and torch.equal(s0, s1) and torch.equal(k0, k1)
            else:
                scale = float(l0.abs().max())
                same = float((l0 - l1).abs().max()) <= 0.05 * scale and float((s0 - s1).abs().max()) <= 0.05 * scale
            if not same or not bool(torch.isfinite(l1).all()):
                failures.append((which, B, S, float((l0 - l1).abs().max()), float((s0 - s1).abs().max()),
                                 float((k0 - k1).abs().max())))
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
