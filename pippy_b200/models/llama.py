"""Llama-family decoder (RMSNorm, RoPE, SwiGLU, optional GQA) as pipeline stages.

A stage owns a contiguous slice of the layers (plus the embedding on the first stage and final norm + LM head on
the last).  Parameter names are those of the whole model (``layers.{global index}...``), so the union of the
stages' ``state_dict()`` keys is the full model's key set: the per-stage checkpoint contract of the reference
(test/test_pipe.py:96-110).

Per layer on CUDA: RMSNorm kernel -> QKV GEMM -> RoPE (in place) + flash attention -> O GEMM with the residual add
in its epilogue -> RMSNorm -> gate/up GEMM -> SwiGLU kernel -> down GEMM with the residual add in its epilogue.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.utils.checkpoint
import torch.nn as nn

from ..ops import functional as pf
from .layers import ROTARY, Embedding, Linear, RMSNorm


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: Optional[int] = None
    ffn_dim: int = 11008
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def kv_heads(self) -> int:
        return self.n_kv_heads or self.n_heads

    @staticmethod
    def llama2_7b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def llama2_13b() -> "LlamaConfig":
        return LlamaConfig(dim=5120, n_layers=40, n_heads=40, ffn_dim=13824)

    @staticmethod
    def tiny(vocab_size=512, dim=256, n_layers=4, n_heads=2, n_kv_heads=None, ffn_dim=512) -> "LlamaConfig":
        return LlamaConfig(vocab_size, dim, n_layers, n_heads, n_kv_heads, ffn_dim)

    def num_params(self) -> int:
        d, f, hd = self.dim, self.ffn_dim, self.head_dim
        per_layer = d * (self.n_heads + 2 * self.kv_heads) * hd + d * d + 3 * d * f + 2 * d
        return self.n_layers * per_layer + 2 * self.vocab_size * d + d

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token: 6 * matmul parameters + causal attention (forward 2*S*d per layer, x3)."""
        d, f, hd = self.dim, self.ffn_dim, self.head_dim
        mm = self.n_layers * (d * (self.n_heads + 2 * self.kv_heads) * hd + d * d + 3 * d * f) + self.vocab_size * d
        attn = self.n_layers * 2 * seq_len * d  # QK^T + PV, causal half, per token
        return 6.0 * mm + 3.0 * attn


class LlamaAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        hd = cfg.head_dim
        self.wqkv = Linear(cfg.dim, (cfg.n_heads + 2 * cfg.kv_heads) * hd, init_std=cfg.init_std, device=device, dtype=dtype)
        self.wo = Linear(cfg.n_heads * hd, cfg.dim, init_std=cfg.init_std, device=device, dtype=dtype)

    def forward(self, h, residual, B: int, S: int):
        cfg = self.cfg
        qkv = self.wqkv(h)
        cos, sin = ROTARY.get(S, cfg.head_dim, cfg.rope_theta, h.device)
        att = pf.rope_attention(qkv, cos, sin, B, S, cfg.n_heads, cfg.kv_heads, cfg.head_dim)
        return self.wo(att, residual=residual)


class LlamaMLP(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None, dtype=None):
        super().__init__()
        self.w_gate_up = Linear(cfg.dim, 2 * cfg.ffn_dim, init_std=cfg.init_std, device=device, dtype=dtype)
        self.w_down = Linear(cfg.ffn_dim, cfg.dim, init_std=cfg.init_std, device=device, dtype=dtype)

    def forward(self, h, residual):
        return self.w_down(pf.swiglu(self.w_gate_up(h)), residual=residual)


class LlamaBlock(nn.Module):
    """One decoder layer, or one half of it when a stage boundary falls between its attention and its MLP
    (``has_attention`` / ``has_ffn``); parameter names are the same either way."""

    def __init__(self, cfg: LlamaConfig, device=None, dtype=None, has_attention: bool = True, has_ffn: bool = True):
        super().__init__()
        self.has_attention, self.has_ffn = has_attention, has_ffn
        if has_attention:
            self.attention_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
            self.attention = LlamaAttention(cfg, device=device, dtype=dtype)
        if has_ffn:
            self.ffn_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
            self.feed_forward = LlamaMLP(cfg, device=device, dtype=dtype)

    def forward(self, x, B: int, S: int):  # x: [B*S, dim]
        if self.has_attention:
            x = self.attention(self.attention_norm(x), x, B, S)
        if self.has_ffn:
            x = self.feed_forward(self.ffn_norm(x), x)
        return x


def layer_range(n_layers: int, stage: int, num_stages: int) -> range:
    """Even split of layers over stages; early stages take the remainder."""
    base, rem = divmod(n_layers, num_stages)
    start = stage * base + min(stage, rem)
    return range(start, start + base + (1 if stage < rem else 0))


def unit_costs(cfg: LlamaConfig, seq_len: int):
    """Relative cost of (attention half, MLP half, head, embedding), from forward FLOPs per token; attention
    FLOPs count double (they run further from the tensor-core peak than the GEMMs) and the head carries the final
    norm and the loss."""
    d, hd = cfg.dim, cfg.head_dim
    attn = 2.0 * d * (cfg.n_heads + 2 * cfg.kv_heads) * hd + 2.0 * d * d + 2.0 * (2.0 * seq_len * d)
    ffn = 6.0 * d * cfg.ffn_dim
    head = 2.0 * d * cfg.vocab_size * 1.35
    return attn, ffn, head, 0.02 * (attn + ffn)


def balanced_partition(cfg: LlamaConfig, num_stages: int, pp_size: int, seq_len: int = 4096, stage_to_rank=None):
    """Cuts the sequence [embed, attn0, mlp0, attn1, mlp1, ..., head] into ``num_stages`` contiguous stages so that
    the most loaded RANK (stage s lives on rank ``stage_to_rank[s]``, by default s % pp_size) carries as little as
    possible.  Boundaries may fall
    between a layer's attention and MLP.  Returns, per stage, a list of ``(layer, has_attention, has_ffn)``.

    With whole layers only, the head (worth most of a layer) always lands on top of a full share of layers; at
    8 ranks x 2 stages that alone makes one rank 16 % slower than the rest."""
    attn, ffn, head, embed = unit_costs(cfg, seq_len)
    units = []  # (cost, layer, kind)
    for i in range(cfg.n_layers):
        units.append((attn, i, "a"))
        units.append((ffn, i, "f"))
    n = len(units)
    if num_stages > n:
        raise ValueError(f"{num_stages} stages for {cfg.n_layers} layers")
    prefix = [0.0]
    for c, _, _ in units:
        prefix.append(prefix[-1] + c)

    def stage_cost(bounds, s):
        c = prefix[bounds[s + 1]] - prefix[bounds[s]]
        if s == 0:
            c += embed
        if s == num_stages - 1:
            c += head
        return c

    def max_rank_load(bounds):
        loads = [0.0] * pp_size
        for s in range(num_stages):
            loads[stage_to_rank[s] if stage_to_rank is not None else s % pp_size] += stage_cost(bounds, s)
        return max(loads), sum(l * l for l in loads)

    total = prefix[-1] + head + embed
    target = total / num_stages
    bounds = [0]
    for s in range(1, num_stages):
        want = s * target - embed
        # nearest unit boundary that keeps every stage non-empty
        lo, hi = bounds[-1] + 1, n - (num_stages - s)
        best = min(range(lo, hi + 1), key=lambda b: abs(prefix[b] - want))
        bounds.append(best)
    bounds.append(n)
    improved = True
    while improved:
        improved = False
        for s in range(1, num_stages):
            for delta in (-1, 1):
                cand = list(bounds)
                cand[s] += delta
                if not (cand[s - 1] < cand[s] < cand[s + 1]):
                    continue
                if max_rank_load(cand) < max_rank_load(bounds):
                    bounds = cand
                    improved = True
    stages = []
    for s in range(num_stages):
        per_layer = {}
        for _, layer, kind in units[bounds[s]:bounds[s + 1]]:
            a, f = per_layer.get(layer, (False, False))
            per_layer[layer] = (a or kind == "a", f or kind == "f")
        stages.append([(layer, a, f) for layer, (a, f) in sorted(per_layer.items())])
    return stages


class LlamaStage(nn.Module):
    """A contiguous slice of the model: ``parts`` lists ``(layer, has_attention, has_ffn)``; the embedding goes with
    ``first`` and the final norm + head with ``last``.  Input: token ids ``[B, S]`` (first stage) or hidden states
    ``[B, S, dim]``; output: hidden states ``[B, S, dim]`` or logits ``[B, S, vocab]``."""

    def __init__(self, cfg: LlamaConfig, layer_ids, first: bool, last: bool, device=None, dtype=None,
                 activation_checkpointing: bool = False):
        super().__init__()
        self.cfg = cfg
        self.first, self.last = first, last
        self.activation_checkpointing = activation_checkpointing
        parts = [(p, True, True) if isinstance(p, int) else tuple(p) for p in layer_ids]
        if first:
            self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim, init_std=cfg.init_std, device=device, dtype=dtype)
        self.layers = nn.ModuleDict({
            str(i): LlamaBlock(cfg, device=device, dtype=dtype, has_attention=a, has_ffn=f) for i, a, f in parts
        })
        if last:
            self.norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
            self.output = Linear(cfg.dim, cfg.vocab_size, init_std=cfg.init_std, device=device, dtype=dtype)

    def forward(self, x):
        if self.first:
            B, S = x.shape
            h = self.tok_embeddings(x)
        else:
            B, S, _ = x.shape
            h = x.reshape(B * S, -1)
        recompute = self.activation_checkpointing and torch.is_grad_enabled() and h.requires_grad
        for blk in self.layers.values():
            if recompute:
                # keep only the block's input; its forward runs again inside the backward (the reference lists
                # activation checkpointing as a TODO, ARCHITECTURE.md:201).  Costs one extra forward per block.
                h = torch.utils.checkpoint.checkpoint(blk, h, B, S, use_reentrant=False)
            else:
                h = blk(h, B, S)
        if self.last:
            h = self.output(self.norm(h))
        return h.view(B, S, -1)


def build_llama_stage(cfg: LlamaConfig, stage: int, num_stages: int, device=None, dtype=torch.bfloat16,
                      pp_size: Optional[int] = None, seq_len: int = 4096, balance: bool = True,
                      stage_to_rank=None, activation_checkpointing: bool = False) -> LlamaStage:
    """Stage ``stage`` of ``num_stages``. With ``balance`` (and a known ``pp_size``) layers are assigned by
    :func:`balanced_partition`; otherwise evenly by whole layers."""
    if balance and pp_size is not None and num_stages > 1:
        parts = balanced_partition(cfg, num_stages, pp_size, seq_len, stage_to_rank)[stage]
    else:
        parts = list(layer_range(cfg.n_layers, stage, num_stages))
    return LlamaStage(cfg, parts, stage == 0, stage == num_stages - 1, device=device, dtype=dtype,
                      activation_checkpointing=activation_checkpointing)


class Llama(LlamaStage):
    """The whole model as one module (a one-stage pipeline)."""

    def __init__(self, cfg: LlamaConfig, device=None, dtype=torch.bfloat16):
        super().__init__(cfg, range(cfg.n_layers), True, True, device=device, dtype=dtype)


def causal_lm_loss(logits, target, ignore_index: int = -100):
    """Mean next-token cross-entropy of one microbatch; ``target`` already holds the shifted labels."""
    return pf.cross_entropy(logits.reshape(-1, logits.shape[-1]), target.reshape(-1), reduction="mean",
                            ignore_index=ignore_index)
