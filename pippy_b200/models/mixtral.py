"""Mixtral-family sparse-MoE decoder (RMSNorm, RoPE theta 1e6, GQA, top-2 routed SwiGLU experts) as pipeline stages.

Dense parts (attention, norms, router, embedding, head) are replicated over the expert-parallel group and their
gradients are averaged across it; each rank holds ``n_experts / ep`` experts of every layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as pf
from ..parallel.ep import EPContext, MoEFeedForward
from .layers import Embedding, Linear, RMSNorm
from .llama import LlamaAttention, LlamaConfig, layer_range


@dataclass
class MixtralConfig(LlamaConfig):
    n_experts: int = 8
    top_k: int = 2
    aux_coef: float = 0.01

    @staticmethod
    def mixtral_16l() -> "MixtralConfig":
        return MixtralConfig(vocab_size=32000, dim=4096, n_layers=16, n_heads=32, n_kv_heads=8, ffn_dim=14336,
                             rope_theta=1e6)

    @staticmethod
    def tiny_moe() -> "MixtralConfig":
        return MixtralConfig(vocab_size=512, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=512, rope_theta=1e6,
                             n_experts=4)


class MixtralBlock(nn.Module):
    def __init__(self, cfg: MixtralConfig, ep: Optional[EPContext], ep_size: int, ep_rank: int, device=None, dtype=None):
        super().__init__()
        self.attention_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
        self.attention = LlamaAttention(cfg, device=device, dtype=dtype)
        self.ffn_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
        self.block_sparse_moe = MoEFeedForward(cfg.dim, cfg.ffn_dim, cfg.n_experts, cfg.top_k, ep, ep_size, ep_rank,
                                               cfg.aux_coef, cfg.init_std, device=device, dtype=dtype)

    def forward(self, x, B: int, S: int):
        x = self.attention(self.attention_norm(x), x, B, S)
        return x + self.block_sparse_moe(self.ffn_norm(x))


class MixtralStage(nn.Module):
    def __init__(self, cfg: MixtralConfig, layer_ids, first: bool, last: bool, ep: Optional[EPContext] = None,
                 ep_size: int = 1, ep_rank: int = 0, device=None, dtype=None):
        super().__init__()
        self.cfg, self.first, self.last = cfg, first, last
        if first:
            self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim, init_std=cfg.init_std, device=device, dtype=dtype)
        self.layers = nn.ModuleDict({
            str(i): MixtralBlock(cfg, ep, ep_size, ep_rank, device=device, dtype=dtype) for i in layer_ids
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
        for blk in self.layers.values():
            h = blk(h, B, S)
        if self.last:
            h = self.output(self.norm(h))
        return h.view(B, S, -1)

    def expert_parameters(self):
        return [p for n, p in self.named_parameters() if n.endswith(".w_gate_up") or n.endswith(".w_down")]

    def dense_parameters(self):
        experts = {id(p) for p in self.expert_parameters()}
        return [p for p in self.parameters() if id(p) not in experts]

    def aux_losses(self):
        return [blk.block_sparse_moe.last_aux_loss for blk in self.layers.values()]


def build_mixtral_stage(cfg: MixtralConfig, stage: int, num_stages: int, ep: Optional[EPContext] = None,
                        ep_size: int = 1, ep_rank: int = 0, device=None, dtype=torch.bfloat16) -> MixtralStage:
    return MixtralStage(cfg, layer_range(cfg.n_layers, stage, num_stages), stage == 0, stage == num_stages - 1, ep,
                        ep_size, ep_rank, device=device, dtype=dtype)
