"""Flat parameter/gradient storage and the fused AdamW that runs over it.

``FlatParams`` moves every parameter of a stage into one contiguous buffer and gives each parameter an fp32
``main_grad`` view into one contiguous gradient buffer: the ops of this package accumulate weight gradients there
(the wgrad GEMM adds in fp32 in its epilogue), the data-parallel reducer works on the same buffer in buckets, and
``FusedAdamW`` updates all of it with a single kernel launch per step.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

import torch
import torch.nn as nn

from .ops import _lib


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class FlatParams:
    """Re-homes ``params`` into one flat buffer per dtype group (a single group is assumed: all params share a
    dtype) and allocates the fp32 gradient buffer. Parameter objects stay the same; only their storage moves."""

    ALIGN = 64  # elements; keeps every parameter 128-byte aligned for TMA and vector accesses

    def __init__(self, params: Iterable[nn.Parameter], grad_dtype: torch.dtype = torch.float32):
        self.params: List[nn.Parameter] = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("FlatParams needs at least one trainable parameter")
        dtype = self.params[0].dtype
        device = self.params[0].device
        if any(p.dtype != dtype or p.device != device for p in self.params):
            raise ValueError("all parameters of a FlatParams group must share dtype and device")
        self.offsets: List[int] = []
        off = 0
        for p in self.params:
            self.offsets.append(off)
            off += _align(p.numel(), self.ALIGN)
        self.numel = off
        self.data = torch.zeros(off, dtype=dtype, device=device)
        self.grad = torch.zeros(off, dtype=grad_dtype, device=device)
        for p, o in zip(self.params, self.offsets):
            view = self.data[o : o + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.grad[o : o + p.numel()].view(p.shape)
            p.grad = None

    def zero_grad(self) -> None:
        self.grad.zero_()
        for p in self.params:
            p.grad = None

    def fold_autograd_grads(self) -> None:
        """Adds gradients that autograd left in ``param.grad`` (ops outside this package, or the CPU path) into
        the flat buffer and clears them, so the flat buffer is the single source of truth."""
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None


class FusedAdamW:
    """AdamW over :class:`FlatParams` buffers. bf16 parameters, fp32 gradients and moments, optional fp32 master
    weights; one kernel launch per flat buffer. Same update rule as ``torch.optim.AdamW``."""

    def __init__(self, flat: FlatParams | Sequence[FlatParams], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, master_weights: bool = False):
        self.groups: List[FlatParams] = [flat] if isinstance(flat, FlatParams) else list(flat)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.step_count = 0
        self.m = [torch.zeros(g.numel, dtype=torch.float32, device=g.data.device) for g in self.groups]
        self.v = [torch.zeros(g.numel, dtype=torch.float32, device=g.data.device) for g in self.groups]
        self.master: List[Optional[torch.Tensor]] = [
            g.data.float() if master_weights else None for g in self.groups
        ]

    def zero_grad(self) -> None:
        for g in self.groups:
            g.zero_grad()

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, zero_grad: bool = False) -> None:
        """One update; gradients are multiplied by ``grad_scale`` first (e.g. 1/microbatches). With
        ``zero_grad=True`` the kernel clears the gradient buffer while it is in cache."""
        self.step_count += 1
        b1, b2 = self.betas
        for g, m, v, master in zip(self.groups, self.m, self.v, self.master):
            g.fold_autograd_grads()
            if g.data.is_cuda and g.data.dtype == torch.bfloat16 and g.grad.dtype == torch.float32:
                rc = _lib.lib().pb_adamw(
                    _lib.ptr(g.data), _lib.ptr(master), _lib.ptr(g.grad), _lib.ptr(m), _lib.ptr(v),
                    _lib.c_ll(g.numel), _lib.c_float(self.lr), _lib.c_float(b1), _lib.c_float(b2),
                    _lib.c_float(self.eps), _lib.c_float(self.weight_decay), _lib.c_int(self.step_count),
                    _lib.c_float(grad_scale), _lib.c_int(int(zero_grad)), _lib.stream_ptr(),
                )
                _lib.check(rc, "pb_adamw")
            else:
                grad = g.grad.float() * grad_scale
                w = master if master is not None else g.data.float()
                m.mul_(b1).add_(grad, alpha=1 - b1)
                v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
                mh = m / (1 - b1 ** self.step_count)
                vh = v / (1 - b2 ** self.step_count)
                w = w * (1 - self.lr * self.weight_decay) - self.lr * mh / (vh.sqrt() + self.eps)
                if master is not None:
                    master.copy_(w)
                g.data.copy_(w.to(g.data.dtype))
                if zero_grad:
                    g.grad.zero_()

    def state_dict(self):
        return {
            "step": self.step_count, "lr": self.lr, "betas": self.betas, "eps": self.eps,
            "weight_decay": self.weight_decay, "m": self.m, "v": self.v, "master": self.master,
        }

    def load_state_dict(self, sd) -> None:
        self.step_count = sd["step"]
        self.lr = sd.get("lr", self.lr)
        self.betas = tuple(sd.get("betas", self.betas))
        self.eps = sd.get("eps", self.eps)
        self.weight_decay = sd.get("weight_decay", self.weight_decay)
        for dst, src in zip(self.m, sd["m"]):
            dst.copy_(src)
        for dst, src in zip(self.v, sd["v"]):
            dst.copy_(src)
        for dst, src in zip(self.master, sd["master"]):
            if dst is not None and src is not None:
                dst.copy_(src)
