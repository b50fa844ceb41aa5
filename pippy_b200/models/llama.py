"""Llama-family decoder (RMSNorm, RoPE, SwiGLU, optional GQA) as pipeline stages.

A stage owns a contiguous slice of the layers (plus the embedding on the first stage and final norm + LM head on
the last).  Parameter names are those of the whole model (``layers.{global index}...``), so the union of the
stages' ``state_dict()`` keys is the full model's key set: the per-stage checkpoint contract of the reference
(test/test_pipe.py:96-110).

Stage boundaries may fall inside a layer (after the attention core, the output projection, the SwiGLU or the down
projection), which is what lets the rank that also carries the LM head be balanced against the others.

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


UNITS = ("a1", "a2", "f1", "f2")


class LlamaAttention(nn.Module):
    """QKV projection + RoPE + causal attention (``core``) and the output projection (``wo``); a stage boundary may
    fall between the two, in which case a module holds only its side's weights."""

    def __init__(self, cfg: LlamaConfig, device=None, dtype=None, has_qkv: bool = True, has_out: bool = True):
        super().__init__()
        self.cfg = cfg
        hd = cfg.head_dim
        if has_qkv:
            self.wqkv = Linear(cfg.dim, (cfg.n_heads + 2 * cfg.kv_heads) * hd, init_std=cfg.init_std, device=device,
                               dtype=dtype)
        if has_out:
            self.wo = Linear(cfg.n_heads * hd, cfg.dim, init_std=cfg.init_std, device=device, dtype=dtype)

    def core(self, h, B: int, S: int):
        cfg = self.cfg
        qkv = self.wqkv(h)
        cos, sin = ROTARY.get(S, cfg.head_dim, cfg.rope_theta, h.device)
        return pf.rope_attention(qkv, cos, sin, B, S, cfg.n_heads, cfg.kv_heads, cfg.head_dim)

    def forward(self, h, residual, B: int, S: int):
        return self.wo(self.core(h, B, S), residual=residual)


class LlamaMLP(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None, dtype=None, has_gate_up: bool = True, has_down: bool = True):
        super().__init__()
        if has_gate_up:
            self.w_gate_up = Linear(cfg.dim, 2 * cfg.ffn_dim, init_std=cfg.init_std, device=device, dtype=dtype)
        if has_down:
            self.w_down = Linear(cfg.ffn_dim, cfg.dim, init_std=cfg.init_std, device=device, dtype=dtype)

    def forward(self, h, residual):
        return self.w_down(pf.swiglu(self.w_gate_up(h)), residual=residual)


class LlamaBlock(nn.Module):
    """One decoder layer, or a contiguous run of its four units when stage boundaries fall inside it:

      a1  attention norm, QKV projection, RoPE, attention      x -> (x, att)
      a2  output projection + residual                         (x, att) -> x
      f1  FFN norm, gate/up projection, SwiGLU                 x -> (x, h)
      f2  down projection + residual                           (x, h) -> x

    Parameter names are those of the whole layer whichever units a module holds."""

    def __init__(self, cfg: LlamaConfig, device=None, dtype=None, has_attention: bool = True, has_ffn: bool = True,
                 units=None):
        super().__init__()
        if units is None:
            units = (("a1", "a2") if has_attention else ()) + (("f1", "f2") if has_ffn else ())
        units = tuple(u for u in UNITS if u in units)
        idx = [UNITS.index(u) for u in units]
        if not units or idx != list(range(idx[0], idx[0] + len(idx))):
            raise ValueError(f"a block holds a contiguous run of {UNITS}, got {units}")
        self.units = units
        self.has_attention, self.has_ffn = "a1" in units and "a2" in units, "f1" in units and "f2" in units
        if "a1" in units:
            self.attention_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
        if "a1" in units or "a2" in units:
            self.attention = LlamaAttention(cfg, device=device, dtype=dtype, has_qkv="a1" in units,
                                            has_out="a2" in units)
        if "f1" in units:
            self.ffn_norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
        if "f1" in units or "f2" in units:
            self.feed_forward = LlamaMLP(cfg, device=device, dtype=dtype, has_gate_up="f1" in units,
                                         has_down="f2" in units)

    def forward(self, x, B: int, S: int, carry=None):
        """``x``: residual stream ``[B*S, dim]``; ``carry``: the attention output or the SwiGLU output handed over
        by the previous stage when this block starts at a2 or f2.  Returns ``x`` (or ``(x, carry)`` when the block
        ends at a1 or f1)."""
        u = self.units
        # norm.fork: the residual operand is the norm's second result, so that the residual branch's gradient is
        # added inside the norm-backward kernel
        if "a1" in u:
            n, x = self.attention_norm.fork(x)
            carry = self.attention.core(n, B, S)
        if "a2" in u:
            x, carry = self.attention.wo(carry, residual=x), None
        if "f1" in u:
            n, x = self.ffn_norm.fork(x)
            carry = pf.swiglu(self.feed_forward.w_gate_up(n))
        if "f2" in u:
            x, carry = self.feed_forward.w_down(carry, residual=x), None
        return x if carry is None else (x, carry)


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


def fine_unit_costs(cfg: LlamaConfig, seq_len: int):
    """Costs of the four units of a layer (see :class:`LlamaBlock`), the head and the embedding, in the units of
    :func:`unit_costs`."""
    attn, ffn, head, embed = unit_costs(cfg, seq_len)
    a2 = 2.0 * cfg.dim * cfg.dim
    f2 = 2.0 * cfg.dim * cfg.ffn_dim
    return {"a1": attn - a2, "a2": a2, "f1": ffn - f2, "f2": f2}, head, embed


# what crossing a stage boundary after a unit costs BOTH neighbouring stages, as a fraction of a layer: a cut after a1
# ships the residual stream and the attention output, a cut after f1 the residual stream and the (2.7 x wider) SwiGLU
# output; the extra transfer and the extra saved tensor are small but not free
_CUT_PENALTY = {"a1": 0.01, "a2": 0.0, "f1": 0.03, "f2": 0.0}


def balanced_partition(cfg: LlamaConfig, num_stages: int, pp_size: int, seq_len: int = 4096, stage_to_rank=None,
                       granularity: str = "unit"):
    """Cuts the sequence [embed, layer units ..., head] into ``num_stages`` contiguous stages so that the most
    loaded RANK (stage s lives on rank ``stage_to_rank[s]``, by default s % pp_size) carries as little as possible.
    ``granularity``: ``"unit"`` allows a boundary after any of a layer's four units, ``"half"`` only between a
    layer's attention and MLP, ``"layer"`` only between layers.  Returns, per stage, a list of ``(layer, units)``.

    With whole layers only, the head (worth most of a layer) always lands on top of a full share of layers; at
    8 ranks x 2 stages that alone makes one rank 16 % slower than the rest, half layers leave 8 %, units about 2 %."""
    fine, head, embed = fine_unit_costs(cfg, seq_len)
    layer_cost = sum(fine.values())
    units = []  # (cost, layer, kind)
    for i in range(cfg.n_layers):
        for kind in UNITS:
            units.append((fine[kind], i, kind))
    n = len(units)
    allowed = {"unit": UNITS, "half": ("a2", "f2"), "layer": ("f2",)}[granularity]

    def can_cut(b):  # a boundary at position b falls after unit b - 1
        return 0 < b < n and units[b - 1][2] in allowed

    if num_stages > sum(1 for b in range(1, n) if can_cut(b)) + 1:
        raise ValueError(f"{num_stages} stages for {cfg.n_layers} layers")
    prefix = [0.0]
    for c, _, _ in units:
        prefix.append(prefix[-1] + c)

    def stage_cost(bounds, s):
        c = prefix[bounds[s + 1]] - prefix[bounds[s]]
        if s == 0:
            c += embed
        else:
            c += _CUT_PENALTY[units[bounds[s] - 1][2]] * layer_cost
        if s == num_stages - 1:
            c += head
        else:
            c += _CUT_PENALTY[units[bounds[s + 1] - 1][2]] * layer_cost
        return c

    def score(bounds):
        loads = [0.0] * pp_size
        for s in range(num_stages):
            loads[stage_to_rank[s] if stage_to_rank is not None else s % pp_size] += stage_cost(bounds, s)
        return max(loads), sum(l * l for l in loads)

    total = prefix[-1] + head + embed
    target = total / num_stages
    cuts = [b for b in range(1, n) if can_cut(b)]
    bounds = [0]
    for s in range(1, num_stages):
        want = s * target - embed
        remaining = num_stages - s  # boundaries still to place after this one, plus the end
        ok = [b for b in cuts if b > bounds[-1] and sum(1 for c in cuts if c > b) >= remaining - 1]
        bounds.append(min(ok, key=lambda b: abs(prefix[b] - want)))
    bounds.append(n)
    # Local search.  Shifting the whole run of boundaries i..j by the same amount moves load from stage i - 1 to
    # stage j (or back) without touching the stages in between, which a single-boundary move cannot do.
    best = score(bounds)
    improved = True
    while improved:
        improved = False
        for i in range(1, num_stages):
            for j in range(i, num_stages):
                for delta in (-1, 1, -2, 2, -3, 3, -4, 4):
                    cand = list(bounds)
                    for q in range(i, j + 1):
                        cand[q] += delta
                    if any(not (cand[q - 1] < cand[q] < cand[q + 1]) or not can_cut(cand[q]) for q in range(i, j + 1)):
                        continue
                    sc = score(cand)
                    if sc < best:
                        bounds, best = cand, sc
                        improved = True
    stages = []
    for s in range(num_stages):
        per_layer = {}
        for _, layer, kind in units[bounds[s]:bounds[s + 1]]:
            per_layer.setdefault(layer, []).append(kind)
        stages.append([(layer, tuple(kinds)) for layer, kinds in sorted(per_layer.items())])
    return stages


def _normalise_parts(layer_ids):
    """Accepts layer numbers, ``(layer, has_attention, has_ffn)`` and ``(layer, units)``; returns ``(layer, units)``."""
    out = []
    for p in layer_ids:
        if isinstance(p, int):
            out.append((p, UNITS))
        elif len(p) == 3:
            out.append((p[0], (("a1", "a2") if p[1] else ()) + (("f1", "f2") if p[2] else ())))
        else:
            out.append((p[0], tuple(p[1])))
    return out


class LlamaStage(nn.Module):
    """A contiguous slice of the model: ``layer_ids`` lists layers, or ``(layer, units)`` for layers the stage holds
    only part of (see :class:`LlamaBlock`); the embedding goes with ``first`` and the final norm + head with
    ``last``.  Input: token ids ``[B, S]`` (first stage) or hidden states ``[B, S, dim]``, plus a second tensor
    ``[B, S, dim or ffn_dim]`` when the stage starts in the middle of an attention or MLP half; output: hidden states
    (plus such a second tensor when it ends in the middle of one) or logits ``[B, S, vocab]``."""

    def __init__(self, cfg: LlamaConfig, layer_ids, first: bool, last: bool, device=None, dtype=None,
                 activation_checkpointing: bool = False):
        super().__init__()
        self.cfg = cfg
        self.first, self.last = first, last
        self.activation_checkpointing = activation_checkpointing
        parts = _normalise_parts(layer_ids)
        if first:
            self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim, init_std=cfg.init_std, device=device, dtype=dtype)
        self.layers = nn.ModuleDict({
            str(i): LlamaBlock(cfg, device=device, dtype=dtype, units=u) for i, u in parts
        })
        if last:
            self.norm = RMSNorm(cfg.dim, cfg.norm_eps, device=device, dtype=dtype)
            self.output = Linear(cfg.dim, cfg.vocab_size, init_std=cfg.init_std, device=device, dtype=dtype)
        carry_dim = {"a1": cfg.n_heads * cfg.head_dim, "f1": cfg.ffn_dim}
        first_unit = parts[0][1][0] if parts else "a1"
        last_unit = parts[-1][1][-1] if parts else "f2"
        # width of the second tensor this stage receives / produces (0 = only the residual stream crosses)
        self.carry_in = 0 if first else {"a2": carry_dim["a1"], "f2": carry_dim["f1"]}.get(first_unit, 0)
        self.carry_out = 0 if last else carry_dim.get(last_unit, 0)

    def forward(self, x, carry=None):
        if self.first:
            B, S = x.shape
            h = self.tok_embeddings(x)
        else:
            B, S, _ = x.shape
            h = x.reshape(B * S, -1)
            if carry is not None:
                carry = carry.reshape(B * S, -1)
        recompute = self.activation_checkpointing and torch.is_grad_enabled() and h.requires_grad
        for blk in self.layers.values():
            if recompute:
                # keep only the block's input; its forward runs again inside the backward (the reference lists
                # activation checkpointing as a TODO, ARCHITECTURE.md:201).  Costs one extra forward per block.
                out = torch.utils.checkpoint.checkpoint(blk, h, B, S, carry, use_reentrant=False)
            else:
                out = blk(h, B, S, carry)
            h, carry = out if isinstance(out, tuple) else (out, None)
        if self.last:
            h = self.output(self.norm(h))
        if carry is not None:
            return h.view(B, S, -1), carry.view(B, S, -1)
        return h.view(B, S, -1)


def build_llama_stage(cfg: LlamaConfig, stage: int, num_stages: int, device=None, dtype=torch.bfloat16,
                      pp_size: Optional[int] = None, seq_len: int = 4096, balance: bool = True,
                      stage_to_rank=None, activation_checkpointing: bool = False) -> LlamaStage:
    """Stage ``stage`` of ``num_stages``. With ``balance`` (True, or a granularity name of
    :func:`balanced_partition`) and a known ``pp_size`` the layers' units are assigned by that function; otherwise
    evenly by whole layers."""
    if balance and pp_size is not None and num_stages > 1:
        parts = balanced_partition(cfg, num_stages, pp_size, seq_len, stage_to_rank,
                                   granularity=balance if isinstance(balance, str) else "unit")[stage]
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
