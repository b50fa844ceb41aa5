"""Llama decoder stages under tensor parallelism with sequence-parallel activations.

Between the parallel regions every rank holds a contiguous shard of the microbatch's tokens (``[T / tp, dim]``):
norms and residuals run on the shard, the QKV and gate/up projections start with the fused all-gather -> GEMM, the
output and down projections end with the fused GEMM -> reduce-scatter (residual added in the same kernel), attention
runs on the rank's own heads over the full sequence.  Pipeline transfers ship the token shard, so each tensor-parallel
rank talks to the same tensor-parallel rank of the neighbouring stage.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as pf
from ..parallel.tp import ColumnParallelLinear, RowParallelLinear, TPContext
from .layers import ROTARY, Embedding, Linear, RMSNorm
from .llama import LlamaConfig, layer_range


class _GatherForHead(torch.autograd.Function):
    """All-gather of the token shards before the (replicated) LM head; every rank then computes the same loss on
    all tokens, so the backward simply keeps this rank's rows."""

    @staticmethod
    def forward(ctx, x_shard, tp):
        group = tp.group
        ctx.rows = x_shard.shape[0]
        ctx.rank = dist.get_rank(group)
        if hasattr(tp, "all_gather_rows") and x_shard.is_cuda:
            return tp.all_gather_rows(x_shard)  # the package's peer-memory all-gather kernel
        out = torch.empty(dist.get_world_size(group) * x_shard.shape[0], x_shard.shape[1], dtype=x_shard.dtype,
                          device=x_shard.device)
        dist.all_gather_into_tensor(out, x_shard.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return g[ctx.rank * ctx.rows : (ctx.rank + 1) * ctx.rows].contiguous(), None


class TPLlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp: Optional[TPContext], tp_size: int, device=None, dtype=None):
        super().__init__()
        assert cfg.n_heads % tp_size == 0 and cfg.kv_heads % tp_size == 0 and cfg.ffn_dim % tp_size == 0
        self.cfg, self.tp_size = cfg, tp_size
        hd = cfg.head_dim
        self.hq, self.hkv = cfg.n_heads // tp_size, cfg.kv_heads // tp_size
        self.attention_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
        self.wqkv = ColumnParallelLinear(cfg.dim, (cfg.n_heads + 2 * cfg.kv_heads) * hd, tp, tp_size, cfg.init_std,
                                         device=device, dtype=dtype)
        self.wo = RowParallelLinear(cfg.n_heads * hd, cfg.dim, tp, tp_size, cfg.init_std, device=device, dtype=dtype)
        self.ffn_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
        self.w_gate_up = ColumnParallelLinear(cfg.dim, 2 * cfg.ffn_dim, tp, tp_size, cfg.init_std, device=device, dtype=dtype)
        self.w_down = RowParallelLinear(cfg.ffn_dim, cfg.dim, tp, tp_size, cfg.init_std, device=device, dtype=dtype)

    def forward(self, x_shard, B: int, S: int):
        cfg = self.cfg
        qkv = self.wqkv(self.attention_norm(x_shard))  # [T, (hq + 2 hkv) * hd] for this rank's heads
        cos, sin = ROTARY.get(S, cfg.head_dim, cfg.rope_theta, x_shard.device)
        att = pf.rope_attention(qkv, cos, sin, B, S, self.hq, self.hkv, cfg.head_dim)
        x_shard = self.wo(att, x_shard)                # reduce-scatter + residual
        h = pf.swiglu(self.w_gate_up(self.ffn_norm(x_shard)))
        return self.w_down(h, x_shard)


class TPLlamaStage(nn.Module):
    """Input: token ids ``[B, S]`` (first stage, same on every tensor-parallel rank) or this rank's token shard
    ``[B*S/tp, dim]``; output: token shard, or logits ``[B, S, vocab]`` on the last stage."""

    def __init__(self, cfg: LlamaConfig, layer_ids, first: bool, last: bool, tp: Optional[TPContext], tp_size: int,
                 tp_rank: int, batch: int, seq_len: int, device=None, dtype=None):
        super().__init__()
        self.cfg, self.first, self.last = cfg, first, last
        self.tp, self.tp_size, self.tp_rank = tp, tp_size, tp_rank
        self.B, self.S = batch, seq_len
        if first:
            self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim, init_std=cfg.init_std, device=device, dtype=dtype)
        self.layers = nn.ModuleDict({str(i): TPLlamaBlock(cfg, tp, tp_size, device=device, dtype=dtype) for i in layer_ids})
        if last:
            self.norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
            self.output = Linear(cfg.dim, cfg.vocab_size, init_std=cfg.init_std, device=device, dtype=dtype)

    def forward(self, x):
        B, S = self.B, self.S
        rows = B * S // self.tp_size
        if self.first:
            flat = x.reshape(-1)[self.tp_rank * rows : (self.tp_rank + 1) * rows]
            h = self.tok_embeddings(flat.view(1, -1))
        else:
            h = x
        for blk in self.layers.values():
            h = blk(h, B, S)
        if self.last:
            h = self.norm(h)
            if self.tp_size > 1:
                h = _GatherForHead.apply(h, self.tp)
            return self.output(h).view(B, S, -1)
        return h


def tp_layer_split(cfg: LlamaConfig, num_stages: int, tp_size: int):
    """Layers per pipeline stage.  Under tensor parallelism a layer costs a rank 1 / tp of its work but the LM head
    (replicated: every rank computes all logits) costs all of it, so the head is worth about ``0.65 * tp`` layers on
    the last stage (measured at TP4 x PP2 on the 13B shape: the head stage took 2.6 layers' time more than the other
    with an even split).  Contiguous counts that minimise the heaviest stage."""
    n = cfg.n_layers
    if num_stages == 1:
        return [n]
    head = 0.65 * tp_size
    share = (n + head) / num_stages
    last = max(1, min(n - (num_stages - 1), round(share - head)))
    base, rem = divmod(n - last, num_stages - 1)
    return [base + (1 if s < rem else 0) for s in range(num_stages - 1)] + [last]


def build_tp_llama_stage(cfg: LlamaConfig, stage: int, num_stages: int, tp: Optional[TPContext], tp_size: int,
                         tp_rank: int, batch: int, seq_len: int, device=None, dtype=torch.bfloat16,
                         balance: bool = True) -> TPLlamaStage:
    if balance and tp_size > 1:
        counts = tp_layer_split(cfg, num_stages, tp_size)
        start = sum(counts[:stage])
        layers = range(start, start + counts[stage])
    else:
        layers = layer_range(cfg.n_layers, stage, num_stages)
    return TPLlamaStage(cfg, layers, stage == 0, stage == num_stages - 1, tp, tp_size, tp_rank, batch, seq_len,
                        device=device, dtype=dtype)
