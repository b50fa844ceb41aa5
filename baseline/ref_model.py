"""Plain PyTorch Llama stage used ONLY by the reference arm of the benchmark.

Stock eager PyTorch: nn.Linear (cuBLAS), F.scaled_dot_product_attention, nn.RMSNorm, F.cross_entropy.  Nothing from
pippy_b200 is imported here: this module stands in for the user model a PiPPy user would bring (the reference
ships no model of its own; its examples wrap HuggingFace decoders of this shape).
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


def rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2 :]
    return torch.cat((-x2, x1), dim=-1)


class Block(nn.Module):
    def __init__(self, dim, n_heads, ffn, eps, dtype, device):
        super().__init__()
        self.n_heads, self.hd = n_heads, dim // n_heads
        self.input_layernorm = nn.RMSNorm(dim, eps=eps, dtype=dtype, device=device)
        self.q_proj = nn.Linear(dim, dim, bias=False, dtype=dtype, device=device)
        self.k_proj = nn.Linear(dim, dim, bias=False, dtype=dtype, device=device)
        self.v_proj = nn.Linear(dim, dim, bias=False, dtype=dtype, device=device)
        self.o_proj = nn.Linear(dim, dim, bias=False, dtype=dtype, device=device)
        self.post_attention_layernorm = nn.RMSNorm(dim, eps=eps, dtype=dtype, device=device)
        self.gate_proj = nn.Linear(dim, ffn, bias=False, dtype=dtype, device=device)
        self.up_proj = nn.Linear(dim, ffn, bias=False, dtype=dtype, device=device)
        self.down_proj = nn.Linear(ffn, dim, bias=False, dtype=dtype, device=device)

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        h = self.input_layernorm(x)
        q = self.q_proj(h).view(B, S, self.n_heads, self.hd).transpose(1, 2)
        k = self.k_proj(h).view(B, S, self.n_heads, self.hd).transpose(1, 2)
        v = self.v_proj(h).view(B, S, self.n_heads, self.hd).transpose(1, 2)
        q = q * cos + rotate_half(q) * sin
        k = k * cos + rotate_half(k) * sin
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.o_proj(a.transpose(1, 2).reshape(B, S, -1))
        h = self.post_attention_layernorm(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class Stage(nn.Module):
    def __init__(self, layer_ids, first, last, vocab, dim, n_heads, ffn, eps, theta, seq_len, dtype, device):
        super().__init__()
        self.first, self.last = first, last
        if first:
            self.embed_tokens = nn.Embedding(vocab, dim, dtype=dtype, device=device)
        self.layers = nn.ModuleDict({str(i): Block(dim, n_heads, ffn, eps, dtype, device) for i in layer_ids})
        if last:
            self.norm = nn.RMSNorm(dim, eps=eps, dtype=dtype, device=device)
            self.lm_head = nn.Linear(dim, vocab, bias=False, dtype=dtype, device=device)
        hd = dim // n_heads
        inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32, device=device) / hd))
        ang = torch.outer(torch.arange(seq_len, dtype=torch.float32, device=device), inv)
        emb = torch.cat((ang, ang), dim=-1)
        self.register_buffer("cos", emb.cos().to(dtype)[None, None], persistent=False)
        self.register_buffer("sin", emb.sin().to(dtype)[None, None], persistent=False)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)

    def forward(self, x):
        if self.first:
            x = self.embed_tokens(x)
        for blk in self.layers.values():
            x = blk(x, self.cos, self.sin)
        if self.last:
            x = self.lm_head(self.norm(x))
        return x
