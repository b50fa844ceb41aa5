"""nn.Module wrappers over ``ops.functional``: the building blocks of the model families in this package."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as pf


class Linear(nn.Module):
    """``y = act(x W^T + b) (+ residual)``; on CUDA bf16 this is one tcgen05 GEMM with a fused epilogue."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, init_std: float = 0.02,
                 device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        self.init_std = init_std
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.weight.device.type != "meta":
            nn.init.normal_(self.weight, mean=0.0, std=self.init_std)
            if self.bias is not None:
                nn.init.zeros_(self.bias)

    def forward(self, x, residual=None, activation: Optional[str] = None):
        return pf.linear(x, self.weight, self.bias, residual=residual, activation=activation)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x):
        return pf.rms_norm(x, self.weight, self.eps)

    def fork(self, x):
        """``(norm(x), x)``; pass the second result to the residual add (see ``pf.rms_norm_fork``)."""
        return pf.rms_norm_fork(x, self.weight, self.eps)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype))

    def forward(self, x):
        return pf.layer_norm(x, self.weight, self.bias, self.eps)


class Embedding(nn.Module):
    """Token embedding with an optional learned position table; returns ``[B*S, H]``."""

    def __init__(self, vocab: int, dim: int, max_positions: int = 0, init_std: float = 0.02, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim, device=device, dtype=dtype))
        self.positions = (
            nn.Parameter(torch.empty(max_positions, dim, device=device, dtype=dtype)) if max_positions > 0 else None
        )
        if self.weight.device.type != "meta":
            nn.init.normal_(self.weight, std=init_std)
            if self.positions is not None:
                nn.init.normal_(self.positions, std=init_std)

    def forward(self, ids):
        S = ids.shape[-1]
        wpe = self.positions[:S] if self.positions is not None and self.positions.shape[0] != S else self.positions
        if wpe is not None and wpe is not self.positions:
            # a sliced view would lose the parameter identity the gradient is written to; use the full table
            wpe = self.positions
        return pf.embedding(ids, self.weight, wpe, S)


class RotaryCache:
    """cos/sin tables per (seq_len, head_dim, theta, device), built once."""

    def __init__(self):
        self._tables = {}

    def get(self, S: int, D: int, theta: float, device):
        key = (S, D, float(theta), str(device))
        t = self._tables.get(key)
        if t is None:
            t = pf.rope_tables(S, D, theta, device)
            self._tables[key] = t
        return t


ROTARY = RotaryCache()
