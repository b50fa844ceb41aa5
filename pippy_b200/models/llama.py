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
    def __init__(self, cfg: LlamaConfig, device=None, dtype=None):
        super().__init__()
        self.attention_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
        self.attention = LlamaAttention(cfg, device=device, dtype=dtype)
        self.ffn_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
        self.feed_forward = LlamaMLP(cfg, device=device, dtype=dtype)

    def forward(self, x, B: int, S: int):  # x: [B*S, dim]
        x = self.attention(self.attention_norm(x), x, B, S)
        return self.feed_forward(self.ffn_norm(x), x)


def layer_range(n_layers: int, stage: int, num_stages: int) -> range:
    """Even split of layers over stages; early stages take the remainder."""
    base, rem = divmod(n_layers, num_stages)
    start = stage * base + min(stage, rem)
    return range(start, start + base + (1 if stage < rem else 0))


class LlamaStage(nn.Module):
    """Layers ``layer_ids`` of the model, with the embedding if ``first`` and the norm + head if ``last``.
    Input: token ids ``[B, S]`` (first stage) or hidden states ``[B, S, dim]``; output: hidden states
    ``[B, S, dim]`` or logits ``[B, S, vocab]``."""

    def __init__(self, cfg: LlamaConfig, layer_ids, first: bool, last: bool, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.first, self.last = first, last
        if first:
            self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim, init_std=cfg.init_std, device=device, dtype=dtype)
        self.layers = nn.ModuleDict({str(i): LlamaBlock(cfg, device=device, dtype=dtype) for i in layer_ids})
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
        for blk in self.layers.values():
            h = blk(h, B, S)
        if self.last:
            h = self.output(self.norm(h))
        return h.view(B, S, -1)


def build_llama_stage(cfg: LlamaConfig, stage: int, num_stages: int, device=None, dtype=torch.bfloat16) -> LlamaStage:
    return LlamaStage(cfg, layer_range(cfg.n_layers, stage, num_stages), stage == 0, stage == num_stages - 1,
                      device=device, dtype=dtype)


class Llama(LlamaStage):
    """The whole model as one module (a one-stage pipeline)."""

    def __init__(self, cfg: LlamaConfig, device=None, dtype=torch.bfloat16):
        super().__init__(cfg, range(cfg.n_layers), True, True, device=device, dtype=dtype)


def causal_lm_loss(logits, target, ignore_index: int = -100):
    """Mean next-token cross-entropy of one microbatch; ``target`` already holds the shifted labels."""
    return pf.cross_entropy(logits.reshape(-1, logits.shape[-1]), target.reshape(-1), reduction="mean",
                            ignore_index=ignore_index)
