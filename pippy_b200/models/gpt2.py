"""GPT-2 family decoder (LayerNorm, learned positions, GELU MLP, tied embedding / LM head) as pipeline stages.

The LM head shares its weight with the token embedding.  When both live on the same rank they are one parameter;
when the pipeline puts them on different ranks each stage holds a copy (``lm_head.weight`` on the last stage) and
:class:`TiedEmbeddingSync` sums the two gradients before the optimizer step, which keeps the copies identical
(the REPLICATE policy of the splitter, done by hand for manual stages).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as pf
from .layers import Embedding, LayerNorm, Linear
from .llama import layer_range


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    dim: int = 768
    n_layers: int = 12
    n_heads: int = 12
    norm_eps: float = 1e-5
    init_std: float = 0.02
    vocab_multiple: int = 128  # the embedding / head are padded to a multiple of this many rows

    @property
    def padded_vocab(self) -> int:
        m = self.vocab_multiple
        return (self.vocab_size + m - 1) // m * m

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @staticmethod
    def small() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(vocab_size=500, n_positions=64, dim=128, n_layers=4, n_heads=2)

    def flops_per_token(self, seq_len: int) -> float:
        d = self.dim
        mm = self.n_layers * 12 * d * d + self.padded_vocab * d
        return 6.0 * mm + 3.0 * self.n_layers * 2 * seq_len * d


class GPT2Block(nn.Module):
    def __init__(self, cfg: GPT2Config, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        d = cfg.dim
        self.ln_1 = LayerNorm(d, cfg.norm_eps, device=device, dtype=dtype)
        self.attn_c_attn = Linear(d, 3 * d, bias=True, init_std=cfg.init_std, device=device, dtype=dtype)
        self.attn_c_proj = Linear(d, d, bias=True, init_std=cfg.init_std, device=device, dtype=dtype)
        self.ln_2 = LayerNorm(d, cfg.norm_eps, device=device, dtype=dtype)
        self.mlp_c_fc = Linear(d, 4 * d, bias=True, init_std=cfg.init_std, device=device, dtype=dtype)
        self.mlp_c_proj = Linear(4 * d, d, bias=True, init_std=cfg.init_std, device=device, dtype=dtype)

    def forward(self, x, B: int, S: int):
        cfg = self.cfg
        qkv = self.attn_c_attn(self.ln_1(x))
        att = pf.rope_attention(qkv, None, None, B, S, cfg.n_heads, cfg.n_heads, cfg.head_dim)
        x = self.attn_c_proj(att, residual=x)
        h = self.mlp_c_fc(self.ln_2(x), activation="gelu_tanh")
        return self.mlp_c_proj(h, residual=x)


class GPT2Stage(nn.Module):
    """Input: token ids [B, S] (first stage) or hidden states [B, S, dim]; output: hidden states or logits
    [B, S, padded_vocab]."""

    def __init__(self, cfg: GPT2Config, layer_ids, first: bool, last: bool, device=None, dtype=None):
        super().__init__()
        self.cfg, self.first, self.last = cfg, first, last
        if first:
            self.wte = Embedding(cfg.padded_vocab, cfg.dim, max_positions=cfg.n_positions, init_std=cfg.init_std,
                                 device=device, dtype=dtype)
        self.h = nn.ModuleDict({str(i): GPT2Block(cfg, device=device, dtype=dtype) for i in layer_ids})
        if last:
            self.ln_f = LayerNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
            if first:
                self.lm_head_weight = None  # tied: use the embedding table itself
            else:
                self.lm_head = Linear(cfg.dim, cfg.padded_vocab, init_std=cfg.init_std, device=device, dtype=dtype)

    def head_weight(self) -> torch.Tensor:
        return self.wte.weight if self.first else self.lm_head.weight

    def forward(self, x):
        if self.first:
            B, S = x.shape
            h = self.wte(x)
        else:
            B, S, _ = x.shape
            h = x.reshape(B * S, -1)
        for blk in self.h.values():
            h = blk(h, B, S)
        if self.last:
            h = pf.linear(self.ln_f(h), self.head_weight())
        return h.view(B, S, -1)


def gpt2_layer_split(cfg: GPT2Config, num_stages: int, head_layers: float = 2.0):
    """Layers per stage.  The LM head over the (padded) vocabulary is heavy next to a 768-wide block: 5.4 blocks'
    worth of FLOPs for GPT-2 small, about 2 blocks' worth of time at 2 x 1024 tokens per microbatch (the small blocks
    are launch-bound, the head is one large GEMM; measured: a stage of 3 blocks 0.030 s per step, 3 blocks + head
    0.050 s).  ``head_layers`` is that weight; the last stage gets correspondingly fewer blocks (it may get none)."""
    n = cfg.n_layers
    if num_stages == 1:
        return [n]
    share = (n + head_layers) / num_stages
    last = max(0, min(n - (num_stages - 1), round(share - head_layers)))
    base, rem = divmod(n - last, num_stages - 1)
    return [base + (1 if s < rem else 0) for s in range(num_stages - 1)] + [last]


def build_gpt2_stage(cfg: GPT2Config, stage: int, num_stages: int, device=None, dtype=torch.bfloat16,
                     balance: bool = False) -> GPT2Stage:
    """``balance`` weighs the LM head when splitting the blocks (:func:`gpt2_layer_split`).  Off by default: at
    GPT-2 small's size a stage's time is the host's launch time, not the GPU's, and the measured step got slower
    with it (4 GPUs, PP4, 16 microbatches of 2 x 1024 tokens: 53.1 ms even, 59.5 ms weighted; the first rank, which
    also feeds the inputs, became the slowest)."""
    if balance:
        counts = gpt2_layer_split(cfg, num_stages)
        start = sum(counts[:stage])
        layers = range(start, start + counts[stage])
    else:
        layers = layer_range(cfg.n_layers, stage, num_stages)
    return GPT2Stage(cfg, layers, stage == 0, stage == num_stages - 1, device=device, dtype=dtype)


def gpt2_loss(cfg: GPT2Config):
    def loss_fn(logits, target):
        return pf.cross_entropy(logits.reshape(-1, logits.shape[-1]), target.reshape(-1), vocab_size=cfg.vocab_size,
                                reduction="mean", ignore_index=-100)

    return loss_fn


class TiedEmbeddingSync:
    """Keeps ``wte.weight`` (first stage) and ``lm_head.weight`` (last stage) identical across pipeline ranks:
    ``broadcast()`` once after initialisation, ``sync_grads()`` after every schedule step. Collective over the
    pipeline group at construction (a two-rank group is created)."""

    def __init__(self, stages, pp_group: Optional[dist.ProcessGroup] = None, last_rank: Optional[int] = None):
        self.first = next((s for s in stages if s.is_first), None)
        self.last = next((s for s in stages if s.is_last), None)
        self.pg = None
        self.active = False
        if not dist.is_initialized():
            return
        world = dist.get_world_size(pp_group)
        num_stages = stages[0].num_stages
        # wrap-around placement unless the caller says where the last stage lives (V shape: on rank 0 too)
        r_first, r_last = 0, ((num_stages - 1) % world if last_rank is None else last_rank)
        from ..comm.p2p import new_groups_worldwide

        ranks = sorted({r_first, r_last})
        global_ranks = [dist.get_global_rank(pp_group, r) if pp_group is not None else r for r in ranks]
        member = r_first != r_last and self._member(pp_group, ranks)
        made = new_groups_worldwide([global_ranks] if member else [])  # every rank of the job takes part
        if r_first == r_last:
            return
        self.pg = made[0] if member else None
        self.src = global_ranks[0] if r_first < r_last else global_ranks[1]
        self.active = self.pg is not None and ((self.first is not None) or (self.last is not None))

    @staticmethod
    def _member(pp_group, ranks) -> bool:
        return dist.get_rank(pp_group) in ranks

    def _param(self):
        if self.first is not None:
            return self.first.submod.wte.weight
        return self.last.submod.lm_head.weight

    @torch.no_grad()
    def broadcast(self) -> None:
        if self.active:
            dist.broadcast(self._param().data, src=self.src, group=self.pg)

    @torch.no_grad()
    def sync_grads(self) -> None:
        if not self.active:
            return
        p = self._param()
        g = getattr(p, "main_grad", None)
        if g is None:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            g = p.grad
        elif p.grad is not None:
            # ops outside this package's kernels (the CPU path) leave their gradient in .grad: fold it in first,
            # or the reduction would miss it and the two copies would drift apart
            g.add_(p.grad.to(g.dtype))
            p.grad = None
        dist.all_reduce(g, group=self.pg)
