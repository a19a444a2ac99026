"""Llama-architecture decoder stack whose linears all run the W4A4 int4 dual-scale path, with
Megatron-style tensor parallelism over the ranks of one node.

This is the harness for the end-to-end configuration (random-init Llama-3.1-8B architecture,
prefill + decode, TP 1/2/4/8): the counterpart of the reference's graph_bench_all.prefill/decode
(ablation/real_int4_kernel/graph_bench_all.py:72-157) around HF's LlamaForCausalLM with every
linear wrapped by PermLinear and the QuaRot online Hadamards installed
(quarot/online_had_install.py:44-58).  Attention, RMSNorm and RoPE stay bf16 torch ops (the
reference leaves them to HF); the seven linears of a layer are four fused W4A4 calls:

    qkv      column-parallel (query/key/value heads split over ranks)
    o_proj   row-parallel   (online partial Hadamard across the rank's heads), all-reduce
    gate+up  column-parallel
    down     row-parallel   (SiLU*up + online Hadamard of the rank's slice + quantiser fused), all-reduce

With tp > 1 the online Hadamards and the per-token activation scales are taken over the rank's
own slice of the sharded axis (a valid rotation / scaling per shard, no collective); the only
collectives are the two all-reduces per layer: NCCL in prefill; in decode either NCCL or, with
fused_allreduce, a sum over NVLink peer memory inside the GEMM kernel's epilogue.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _lib, ops, quarot, sharding, synthetic


@dataclass
class DecoderConfig:
    hidden_size: int = 4096
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    vocab_size: int = 128256
    rope_theta: float = 500000.0
    rms_norm_eps: float = 1e-5
    online_hadamard: bool = True


LLAMA31_8B = DecoderConfig()


class W4A4Linear:
    """Packed int4 weight + DualQuant scales (+ optional online Hadamard) of one linear shard."""

    def __init__(self, N: int, K: int, device, gen: torch.Generator, had: Optional[ops.Hadamard] = None,
                 keep_codes: bool = False, gen_a: Optional[torch.Generator] = None):
        """gen_a: generator of the input-channel scale; the shards of a column-parallel linear pass
        one that is seeded alike on every rank (they share their input channels, hence the scale)."""
        w = (torch.randn(N, K, generator=gen, device=device) * 0.02).to(torch.bfloat16)
        codes, sw = ops.quant_w_int4(w)
        self.pw = ops.pack_w_int4(codes, sw)
        # checkers rebuild the layer on the CPU from the unpacked codes and group scales
        self.codes, self.sw = (codes, sw) if keep_codes else (None, None)
        del w, codes, sw
        self.r = torch.exp(torch.randn(N, generator=gen, device=device) * 0.3).half().float()
        c = torch.exp(torch.randn(K, generator=gen_a if gen_a is not None else gen, device=device) * 0.3).half().float()
        self.a = 1.0 / c
        self.had = had
        self.N, self.K = N, K
        self._scratch = {}

    def _scratch_for(self, M: int, device):
        buf = self._scratch.get(M)
        if buf is None:
            buf = torch.empty(max(ops.linear_scratch_bytes(M, self.N, self.K), 256), dtype=torch.uint8,
                              device=device)
            self._scratch[M] = buf
        return buf

    # From this many tokens on the linears run on the FP8-path GEMM with the weight's byte form kept
    # next to the 4-bit artefact (N * K bytes more per weight; same results bit for bit).
    PREFILL_TOKENS = 512

    def _gemm(self, codes, sx, out_dtype=torch.bfloat16, residual=None):
        if codes.dtype == torch.uint8:
            return ops.gemm_w4a4_int4_e4m3(codes, sx, self.pw.bytes_e4m3(), self.pw, self.r, out_dtype=out_dtype,
                                           residual=residual)
        return ops.gemm_w4a4_int4(codes, sx, self.pw, self.r, out_dtype=out_dtype, residual=residual)

    def normed(self, x: torch.Tensor, norm_weight: torch.Tensor, eps: float,
               out_dtype=torch.bfloat16) -> torch.Tensor:
        """RMSNorm(x) -> this linear, the norm fused into the activation quantiser."""
        codes, sx = ops.quant_act_int4_rmsnorm(x, norm_weight, eps, self.a, False,
                                               e4m3=x.shape[0] >= self.PREFILL_TOKENS)
        return self._gemm(codes, sx, out_dtype)

    def __call__(self, x: torch.Tensor, out_dtype=torch.bfloat16, ar=None, residual=None) -> torch.Tensor:
        """ar: an ops.AllReduceContext -> the cross-rank sum happens inside the GEMM (M <= 16).
        residual: [M, N] bf16 -> returns residual + linear, the sum formed in the GEMM epilogue."""
        if ar is not None:
            codes, sx = ops.quant_act_int4(x, self.a, self.had, False)
            return ops.gemm_w4a4_int4_ar(codes, sx, self.pw, self.r, ar, out_dtype=out_dtype, residual=residual)
        big = x.shape[0] >= self.PREFILL_TOKENS
        if residual is not None or big:
            codes, sx = ops.quant_act_int4(x, self.a, self.had, False, e4m3=big)
            return self._gemm(codes, sx, out_dtype, residual)
        return ops.linear_w4a4_int4(x, self.a, self.had, self.pw, self.r, out_dtype=out_dtype,
                                    scale_fp16=False, scratch=self._scratch_for(x.shape[0], x.device))

    def gated(self, gate: torch.Tensor, up: torch.Tensor, out_dtype=torch.bfloat16, ar=None,
              residual=None) -> torch.Tensor:
        big = ar is None and gate.shape[0] >= self.PREFILL_TOKENS
        codes, sx = ops.quant_act_int4_gated(gate, up, self.a, self.had, False, e4m3=big)
        if ar is not None:
            return ops.gemm_w4a4_int4_ar(codes, sx, self.pw, self.r, ar, out_dtype=out_dtype, residual=residual)
        return self._gemm(codes, sx, out_dtype, residual)


def _rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return F.rms_norm(x, (x.shape[-1],), weight, eps)


def _rope_tables(cfg: DecoderConfig, max_pos: int, device):
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=device).float() / cfg.head_dim))
    ang = torch.arange(max_pos, device=device).float()[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)


def _apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x [B, H, S, D]; cos/sin [S, D]
    d = x.shape[-1] // 2
    rot = torch.cat([-x[..., d:], x[..., :d]], dim=-1)
    return x * cos + rot * sin


_HAD_MATRICES = {}


def _shared_hadamard_matrix(hk, kk: int, device):
    """One device copy of the K x K Hadamard factor per (order, device), shared by all layers: the
    quantiser skips its table upload when consecutive calls bring the same matrix pointer."""
    if hk is None:
        return None
    key = (int(kk), str(device))
    if key not in _HAD_MATRICES:
        _HAD_MATRICES[key] = hk.to(device=device, dtype=torch.float32).contiguous()
    return _HAD_MATRICES[key]


class DecoderLayer:
    def __init__(self, cfg: DecoderConfig, tp: int, device, gen: torch.Generator, keep_codes: bool = False,
                 shared: Optional[torch.Generator] = None):
        self.cfg, self.tp = cfg, tp
        hd = cfg.head_dim
        self.hq = cfg.num_attention_heads // tp
        self.hkv = cfg.num_key_value_heads // tp
        inter = cfg.intermediate_size // tp
        had_o = had_d = None
        if cfg.online_hadamard:
            if self.hq > 1:
                had_o = ops.Hadamard(_lib.HAD_PARTIAL, 1, hd, quarot.partial_hadamard_scale(self.hq), None)
            hk, kk = quarot.get_hadK(inter)
            had_d = ops.Hadamard(_lib.HAD_FULL, kk, 0, quarot.full_hadamard_scale(inter),
                                 _shared_hadamard_matrix(hk, kk, device))
        self.qkv = W4A4Linear((self.hq + 2 * self.hkv) * hd, cfg.hidden_size, device, gen, None, keep_codes, shared)
        self.o = W4A4Linear(cfg.hidden_size, self.hq * hd, device, gen, had_o, keep_codes)
        self.gate_up = W4A4Linear(2 * inter, cfg.hidden_size, device, gen, None, keep_codes, shared)
        self.down = W4A4Linear(cfg.hidden_size, inter, device, gen, had_d, keep_codes)
        self.inter = inter
        self.ln1 = torch.ones(cfg.hidden_size, dtype=torch.bfloat16, device=device)
        self.ln2 = torch.ones(cfg.hidden_size, dtype=torch.bfloat16, device=device)
        self.k_cache = self.v_cache = None

    def alloc_cache(self, batch: int, max_len: int, device):
        shape = (batch, self.hkv, max_len, self.cfg.head_dim)
        self.k_cache = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.v_cache = torch.zeros(shape, dtype=torch.bfloat16, device=device)

    def forward(self, x, cos, sin, pos0: int, pos_t: Optional[torch.Tensor], mask, group, ar=None,
                rope_tabs=None):
        """x [B, S, hidden] bf16.  Prefill: pos0 = 0, pos_t None (causal).  Decode: S = 1, the
        cache position comes from the device tensor pos_t and `mask` hides the unwritten tail."""
        cfg = self.cfg
        B, S, Hd = x.shape
        hd = cfg.head_dim
        qkv = self.qkv.normed(x.reshape(B * S, Hd), self.ln1, cfg.rms_norm_eps)
        if rope_tabs is not None:
            # RoPE + cache write in one launch; attention reads K / V straight from the cache
            if pos_t is not None:
                q = ops.rope_kv_append(qkv, rope_tabs[0], rope_tabs[1], pos_t, self.hq, self.hkv,
                                       self.k_cache, self.v_cache, S)
                attn = F.scaled_dot_product_attention(q, self.k_cache, self.v_cache, attn_mask=mask,
                                                      enable_gqa=True)
            else:
                q = ops.rope_kv_append(qkv, rope_tabs[0], rope_tabs[1], pos0, self.hq, self.hkv,
                                       self.k_cache, self.v_cache, S)
                attn = F.scaled_dot_product_attention(q, self.k_cache[:, :, pos0 : pos0 + S],
                                                      self.v_cache[:, :, pos0 : pos0 + S], is_causal=True,
                                                      enable_gqa=True)
            attn = attn.transpose(1, 2).reshape(B * S, self.hq * hd)
            return self._after_attention(x, attn, group, ar)
        qkv = qkv.reshape(B, S, self.hq + 2 * self.hkv, hd)
        q = qkv[:, :, : self.hq].transpose(1, 2)
        k = qkv[:, :, self.hq : self.hq + self.hkv].transpose(1, 2)
        v = qkv[:, :, self.hq + self.hkv :].transpose(1, 2)
        q, k = _apply_rope(q, cos, sin), _apply_rope(k, cos, sin)
        rep = self.hq // self.hkv  # grouped-query attention: expand K/V heads for the fused kernels
        if pos_t is None:
            self.k_cache[:, :, pos0 : pos0 + S] = k
            self.v_cache[:, :, pos0 : pos0 + S] = v
            attn = F.scaled_dot_product_attention(q, k.repeat_interleave(rep, dim=1),
                                                  v.repeat_interleave(rep, dim=1), is_causal=True)
        else:
            self.k_cache.index_copy_(2, pos_t, k)
            self.v_cache.index_copy_(2, pos_t, v)
            attn = F.scaled_dot_product_attention(q, self.k_cache, self.v_cache, attn_mask=mask,
                                                  enable_gqa=True)
        attn = attn.transpose(1, 2).reshape(B * S, self.hq * hd)
        return self._after_attention(x, attn, group, ar)

    def forward_token_sharded(self, x, B: int, S: int, group, rope_tabs, codes, sx, xc=None):
        """Prompt pass under tensor parallelism with the residual stream sharded over tokens: x is
        this rank's [B * S / tp, hidden] slice (ranks own consecutive blocks of tokens).  RMSNorm
        and the activation quantiser run on the slice, the codes (one byte per element) and token
        scales are all-gathered into `codes` [B * S, hidden] / `sx` [B * S], the column-parallel
        linears and the attention of this rank's heads see every token, and the partial outputs of
        the row-parallel linears come back through a reduce-scatter.  Against all-reduce + replicated
        norms: three quarters of the bytes on the wire and 1/tp of the element-wise work.
        xc: an ops.ExchangeContext -> the exchange runs over peer memory instead of NCCL: the
        row-parallel GEMMs push their output tiles into the owners' partial buffers from their
        epilogues, the owners add them onto x (in place) and push their codes to every rank."""
        if xc is not None:
            return self._forward_token_sharded_peer(x, B, S, rope_tabs, xc)
        cfg = self.cfg
        Tq, Hd = x.shape
        T = B * S
        hd = cfg.head_dim
        e4m3 = codes.dtype == torch.uint8
        c_sh, s_sh = ops.quant_act_int4_rmsnorm(x, self.ln1, cfg.rms_norm_eps, self.qkv.a, False, e4m3=e4m3)
        dist.all_gather_into_tensor(codes, c_sh, group=group)
        dist.all_gather_into_tensor(sx, s_sh, group=group)
        qkv = self.qkv._gemm(codes, sx)
        q = ops.rope_kv_append(qkv, rope_tabs[0], rope_tabs[1], 0, self.hq, self.hkv, self.k_cache, self.v_cache, S)
        attn = F.scaled_dot_product_attention(q, self.k_cache[:, :, :S], self.v_cache[:, :, :S], is_causal=True,
                                              enable_gqa=True)
        o = self.o(attn.transpose(1, 2).reshape(T, self.hq * hd))
        o_sh = torch.empty(Tq, Hd, dtype=o.dtype, device=o.device)
        dist.reduce_scatter_tensor(o_sh, o, group=group)
        x = x + o_sh
        c_sh, s_sh = ops.quant_act_int4_rmsnorm(x, self.ln2, cfg.rms_norm_eps, self.gate_up.a, False, e4m3=e4m3)
        dist.all_gather_into_tensor(codes, c_sh, group=group)
        dist.all_gather_into_tensor(sx, s_sh, group=group)
        gu = self.gate_up._gemm(codes, sx)
        d = self.down.gated(gu[:, : self.inter], gu[:, self.inter :])
        d_sh = torch.empty(Tq, Hd, dtype=d.dtype, device=d.device)
        dist.reduce_scatter_tensor(d_sh, d, group=group)
        return x + d_sh

    def _forward_token_sharded_peer(self, x, B: int, S: int, rope_tabs, xc):
        cfg = self.cfg
        T = B * S
        c_sh, s_sh = ops.quant_act_int4_rmsnorm(x, self.ln1, cfg.rms_norm_eps, self.qkv.a, False, e4m3=True)
        xc.push(c_sh, s_sh)
        xc.barrier()  # every rank's codes have landed here
        qkv = self.qkv._gemm(xc.codes, xc.sx)
        q = ops.rope_kv_append(qkv, rope_tabs[0], rope_tabs[1], 0, self.hq, self.hkv, self.k_cache, self.v_cache, S)
        attn = F.scaled_dot_product_attention(q, self.k_cache[:, :, :S], self.v_cache[:, :, :S], is_causal=True,
                                              enable_gqa=True)
        attn = attn.transpose(1, 2).reshape(T, self.hq * cfg.head_dim)
        c_o, s_o = ops.quant_act_int4(attn, self.o.a, self.o.had, False, e4m3=True)
        ops.gemm_w4a4_int4_e4m3_scatter(c_o, s_o, self.o.pw.bytes_e4m3(), self.o.pw, self.o.r, xc)
        xc.barrier()  # every rank's partial rows for this rank's tokens have landed
        xc.add_partials(x)
        c_sh, s_sh = ops.quant_act_int4_rmsnorm(x, self.ln2, cfg.rms_norm_eps, self.gate_up.a, False, e4m3=True)
        xc.push(c_sh, s_sh)
        xc.barrier()
        gu = self.gate_up._gemm(xc.codes, xc.sx)
        c_d, s_d = ops.quant_act_int4_gated(gu[:, : self.inter], gu[:, self.inter :], self.down.a, self.down.had,
                                            False, e4m3=True)
        ops.gemm_w4a4_int4_e4m3_scatter(c_d, s_d, self.down.pw.bytes_e4m3(), self.down.pw, self.down.r, xc)
        xc.barrier()
        xc.add_partials(x)
        return x

    def _after_attention(self, x, attn, group, ar):
        """o_proj, residual, MLP, residual."""
        cfg = self.cfg
        B, S, Hd = x.shape
        fused = ar if (ar is not None and self.tp > 1 and B * S <= 16) else None
        if self.tp == 1:
            # one GPU: the residual additions ride in the epilogues of o_proj and down_proj
            x = self.o(attn, residual=x.reshape(B * S, Hd).contiguous()).reshape(B, S, Hd)
            gu = self.gate_up.normed(x.reshape(B * S, Hd), self.ln2, cfg.rms_norm_eps)
            return self.down.gated(gu[:, : self.inter], gu[:, self.inter :],
                                   residual=x.reshape(B * S, Hd)).reshape(B, S, Hd)
        if fused is not None:
            # decode batch: the cross-rank sum and the residual addition both happen as the row-parallel
            # GEMM stores its rows
            x2 = self.o(attn, ar=fused, residual=x.reshape(B * S, Hd).contiguous())
            gu = self.gate_up.normed(x2, self.ln2, cfg.rms_norm_eps)
            return self.down.gated(gu[:, : self.inter], gu[:, self.inter :], ar=fused,
                                   residual=x2).reshape(B, S, Hd)
        o = self.o(attn)
        dist.all_reduce(o, group=group)
        x = x + o.reshape(B, S, Hd)
        gu = self.gate_up.normed(x.reshape(B * S, Hd), self.ln2, cfg.rms_norm_eps)
        d = self.down.gated(gu[:, : self.inter], gu[:, self.inter :])
        dist.all_reduce(d, group=group)
        return x + d.reshape(B, S, Hd)


class Decoder:
    def __init__(self, cfg: DecoderConfig, device, tp: int = 1, rank: int = 0, seed: int = 0, group=None,
                 fused_allreduce: bool = False, keep_codes: bool = False, token_sharded_prefill: bool = True,
                 prefill_exchange: str = "peer"):
        """fused_allreduce: decode steps sum the row-parallel linears' partial outputs inside the
        GEMM kernel over NVLink peer memory instead of calling NCCL (prefill keeps NCCL).
        token_sharded_prefill: with tp > 1, prompts whose token count divides by tp keep the residual
        stream sharded over tokens (reduce-scatter / all-gather of codes) instead of all-reducing it.
        prefill_exchange: "peer" - that exchange runs in this library's kernels over NVLink peer memory
        (needs tokens / tp a multiple of 256 and at least 512 tokens, else NCCL carries it); "nccl"."""
        if prefill_exchange not in ("peer", "nccl"):
            raise ValueError("prefill_exchange must be 'peer' or 'nccl'")
        assert cfg.num_key_value_heads % tp == 0 and cfg.intermediate_size % (tp * 128) == 0
        self.cfg, self.tp, self.rank, self.group, self.device = cfg, tp, rank, group, device
        self.token_sharded_prefill = token_sharded_prefill
        self.prefill_exchange = prefill_exchange
        self._exchange = {}
        self.ar = None
        if fused_allreduce and tp > 1:
            self.ar = ops.AllReduceContext(group if group is not None else dist.group.WORLD, device,
                                           capacity_floats=16 * cfg.hidden_size)
        gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)  # each rank: its own shard
        shared = torch.Generator(device=device).manual_seed(seed)             # replicated tensors
        self.embed = (torch.randn(cfg.vocab_size, cfg.hidden_size, generator=shared, device=device) * 0.02).to(torch.bfloat16)
        self.lm_head = (torch.randn(cfg.vocab_size, cfg.hidden_size, generator=shared, device=device) * 0.02).to(torch.bfloat16)
        self.norm = torch.ones(cfg.hidden_size, dtype=torch.bfloat16, device=device)
        self.layers = [DecoderLayer(cfg, tp, device, gen, keep_codes, shared) for _ in range(cfg.num_hidden_layers)]
        self.max_len = 0

    def alloc_cache(self, batch: int, max_len: int):
        self.max_len = max_len
        for layer in self.layers:
            layer.alloc_cache(batch, max_len, self.device)
        self.cos, self.sin = _rope_tables(self.cfg, max_len, self.device)

    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, S] -> logits of the last position [B, vocab]."""
        B, S = ids.shape
        return self._prefill_tail(self._prefill_body(ids), B, S)

    def _token_sharded(self, B: int, S: int) -> bool:
        return self.tp > 1 and self.token_sharded_prefill and (B * S) % self.tp == 0

    def _peer_exchange(self, B: int, S: int) -> bool:
        return (self._token_sharded(B, S) and self.prefill_exchange == "peer" and
                sharding.peer_exchange_fits(B * S, self.tp, self.cfg.hidden_size, W4A4Linear.PREFILL_TOKENS))

    def _prefill_body(self, ids: torch.Tensor) -> torch.Tensor:
        """The decoder layers of a prompt pass: kernels on the current stream only - no host
        synchronisation and, on one GPU or with the peer-memory exchange, no library collective - so
        that it can be captured in a CUDA graph.  Returns the last positions' hidden states [B, hidden]
        or, token-sharded, this rank's slice of the residual stream."""
        cfg = self.cfg
        B, S = ids.shape
        if not self._token_sharded(B, S):
            x = self.embed[ids]
            cos, sin = self.cos[:S], self.sin[:S]
            for layer in self.layers:
                x = layer.forward(x, cos, sin, 0, None, None, self.group, rope_tabs=(self.cos, self.sin))
            return x[:, -1]
        T, Hd = B * S, cfg.hidden_size
        lo, hi = sharding.token_shard(T, self.tp, self.rank)
        Tq = hi - lo
        x = self.embed[ids.reshape(-1)[lo:hi]]
        e4m3 = T >= W4A4Linear.PREFILL_TOKENS
        xc = None
        if self._peer_exchange(B, S):
            xc = self._exchange.get(Tq)
            if xc is None:  # collective: every rank reaches this with the same Tq
                xc = self._exchange[Tq] = ops.ExchangeContext(
                    self.group if self.group is not None else dist.group.WORLD, self.device, Tq, Hd)
            codes = sx = None
        else:
            codes = torch.empty(T, Hd, dtype=torch.uint8 if e4m3 else torch.int8, device=self.device)
            sx = torch.empty(T, dtype=torch.float32, device=self.device)
        for layer in self.layers:
            x = layer.forward_token_sharded(x, B, S, self.group, (self.cos, self.sin), codes, sx, xc)
        return x

    def _prefill_tail(self, x: torch.Tensor, B: int, S: int) -> torch.Tensor:
        """Final norm and output projection of the last positions (collected from their owners first
        when the residual stream is token-sharded)."""
        cfg = self.cfg
        if self._token_sharded(B, S):
            if self._peer_exchange(B, S):
                _lib.device_status(self.device.index)  # a barrier that gave up must not pass as a result
            # the last position of every sequence lives on exactly one rank: the others contribute zeros
            last = torch.zeros(B, cfg.hidden_size, dtype=torch.bfloat16, device=self.device)
            mine = sharding.last_token_rows(B, S, self.tp, self.rank)
            if mine:
                rows = torch.tensor([row for _, row in mine], device=self.device)
                last[torch.tensor([b for b, _ in mine], device=self.device)] = x[rows]
            dist.all_reduce(last, group=self.group)
            x = last
        return _rms_norm(x, self.norm, cfg.rms_norm_eps) @ self.lm_head.T

    def capture_prefill(self, ids: torch.Tensor):
        """The prompt pass for prompts of ids' shape as a CUDA graph (the reference's harness times its
        prompt pass the same way, ablation/real_int4_kernel/graph_bench_all.py:72-92): returns
        run(new_ids=None) -> logits, which copies new_ids into the captured input, replays the layers
        and finishes with the eager tail.  Where the layers hold a library collective (tensor
        parallelism over NCCL) nothing is captured and run() is the eager prefill.  With the
        peer-memory exchange all ranks must capture and replay together."""
        B, S = ids.shape
        if self.tp > 1 and not self._peer_exchange(B, S):
            return lambda new_ids=None: self.prefill(ids if new_ids is None else new_ids)
        static_ids = ids.clone()
        cur = torch.cuda.current_stream(self.device)
        side = torch.cuda.Stream(device=self.device)
        with torch.no_grad():
            side.wait_stream(cur)
            with torch.cuda.stream(side):  # lazy set-up (byte forms of the weights, exchange buffers) happens here
                self._prefill_body(static_ids)
            cur.wait_stream(side)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self._prefill_body(static_ids)

        def run(new_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
            if new_ids is not None:
                static_ids.copy_(new_ids)
            graph.replay()
            with torch.no_grad():
                return self._prefill_tail(out, B, S)

        run.graph = graph
        return run

    def decode_step(self, ids: torch.Tensor, pos_t: torch.Tensor) -> torch.Tensor:
        """ids [B] (one token per sequence), pos_t: int64 device tensor [1] with the cache position.
        Everything is indexed through pos_t, so the step can be captured in a CUDA graph."""
        x = self.embed[ids].unsqueeze(1)
        cos = self.cos.index_select(0, pos_t)
        sin = self.sin.index_select(0, pos_t)
        # additive mask over the unwritten tail of the cache, built once per step (a boolean mask
        # would be converted by the attention call in every layer)
        hidden = torch.arange(self.max_len, device=self.device) > pos_t
        mask = torch.zeros(self.max_len, dtype=torch.bfloat16, device=self.device).masked_fill_(hidden, float("-inf"))
        mask = mask.view(1, 1, 1, self.max_len)
        for layer in self.layers:
            x = layer.forward(x, cos, sin, 0, pos_t, mask, self.group, self.ar, rope_tabs=(self.cos, self.sin))
        x = _rms_norm(x[:, 0], self.norm, self.cfg.rms_norm_eps)
        return x @ self.lm_head.T


def linear_weight_bytes(cfg: DecoderConfig) -> int:
    """Algorithmic int4 weight bytes (codes + fp16 group scales) of all decoder linears."""
    hd = cfg.head_dim
    per_layer = 0
    for N, K in (((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * hd, cfg.hidden_size),
                 (cfg.hidden_size, cfg.num_attention_heads * hd),
                 (2 * cfg.intermediate_size, cfg.hidden_size),
                 (cfg.hidden_size, cfg.intermediate_size)):
        per_layer += N * K // 2 + N * (K // 128) * 2
    return per_layer * cfg.num_hidden_layers
