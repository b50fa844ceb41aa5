"""Expert parallelism for sparse MoE layers (top-k routing, SwiGLU experts) on fused NVLink kernels.

Per MoE layer and microbatch, on every rank of the expert-parallel group:

  route      router GEMM (tcgen05) -> softmax / top-k / load-balance statistics on the tiny [T, E] tensor
  dispatch   ONE kernel permutes the token rows and stores each straight into the receive buffer of the rank that
             owns the expert, grouped by expert (``csrc/moe.cu``: P2P stores, flag handshakes)
  experts    the local experts run the package's GEMM / SwiGLU kernels on their contiguous row groups
  combine    ONE kernel pulls every token's k expert rows back from the owning ranks, un-permutes and forms the
             weighted sum in fp32

Backward swaps the roles: the gradient of ``combine`` is a dispatch of ``w * dy`` rows (plus a row-dot kernel for
the router-weight gradients), the gradient of ``dispatch`` is a combine with unit weights.  Only the [world, E]
assignment counts travel through NCCL (32 bytes per rank).  The reference has no expert parallelism; its MoE example
places whole experts on pipeline stages (examples/mixture_of_experts/dist_moe.py:43-59).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import _lib
from ..ops import functional as pf


class EPContext:
    """Peer-mapped workspaces of one expert-parallel group, shared by all MoE layers (calls are stream ordered)."""

    def __init__(self, group: Optional[dist.ProcessGroup], max_tokens: int, hidden: int, top_k: int = 2, device=None,
                 ctas: int = 96):
        from ..comm.symm import SymmetricBuffer

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.hidden, self.top_k, self.ctas = hidden, top_k, ctas
        self.capacity = self.world * max_tokens * top_k  # worst case: every assignment of every rank lands here
        nbytes = self.capacity * hidden * 2
        self.recv = SymmetricBuffer(nbytes, group, self.device)
        self.ybuf = SymmetricBuffer(nbytes, group, self.device)
        self.flags_d = SymmetricBuffer(4096, group, self.device)
        self.flags_c = SymmetricBuffer(4096, group, self.device)
        self.counter = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.recv_ptrs = torch.tensor(self.recv.ptrs, dtype=torch.int64, device=self.device)
        self.y_ptrs = torch.tensor(self.ybuf.ptrs, dtype=torch.int64, device=self.device)
        self.epoch_d = 0
        self.epoch_c = 0

    def _flags(self, buf):
        arr = (ctypes.POINTER(ctypes.c_int) * self.world)()
        for i, ptr in enumerate(buf.ptrs):
            arr[i] = ctypes.cast(ctypes.c_void_p(ptr), ctypes.POINTER(ctypes.c_int))
        return arr

    def recv_rows(self, n: int) -> torch.Tensor:
        return self.recv.tensor(torch.bfloat16, n * self.hidden).view(n, self.hidden)

    def y_rows(self, n: int) -> torch.Tensor:
        return self.ybuf.tensor(torch.bfloat16, n * self.hidden).view(n, self.hidden)

    def dispatch(self, x, expert, slot, dst_base, scale, experts_per_rank):
        T = x.shape[0]
        self.epoch_d += 1
        rc = _lib.lib().pb_moe_dispatch(
            _lib.ptr(x), _lib.ptr(expert), _lib.ptr(slot), _lib.ptr(dst_base), _lib.ptr(scale),
            _lib.ptr(self.recv_ptrs), _lib.c_int(T), _lib.c_int(self.top_k), _lib.c_int(self.hidden),
            _lib.c_int(experts_per_rank), self._flags(self.flags_d), _lib.ptr(self.counter),
            _lib.ptr(_lib.err_word(x.device)), _lib.c_int(self.rank), _lib.c_int(self.world),
            _lib.c_int(self.epoch_d), _lib.c_int(self.ctas), _lib.stream_ptr())
        _lib.check(rc, "pb_moe_dispatch")

    def combine(self, out, expert, slot, dst_base, weight, save, experts_per_rank):
        T = out.shape[0]
        self.epoch_c += 1
        rc = _lib.lib().pb_moe_combine(
            _lib.ptr(out), _lib.ptr(expert), _lib.ptr(slot), _lib.ptr(dst_base), _lib.ptr(weight),
            _lib.ptr(self.y_ptrs), _lib.ptr(save), _lib.c_int(T), _lib.c_int(self.top_k), _lib.c_int(self.hidden),
            _lib.c_int(experts_per_rank), self._flags(self.flags_c), _lib.ptr(self.counter[1:]),
            _lib.ptr(_lib.err_word(out.device)), _lib.c_int(self.rank), _lib.c_int(self.world),
            _lib.c_int(self.epoch_c), _lib.c_int(self.ctas), _lib.stream_ptr())
        _lib.check(rc, "pb_moe_combine")


class _Plan:
    """Routing result of one layer call, shared by the dispatch and combine autograd nodes."""

    def __init__(self, ep: EPContext, expert: torch.Tensor, n_experts: int):
        self.ep = ep
        self.expert = expert  # int32 [T*k]
        self.n_experts = n_experts
        self.experts_per_rank = n_experts // ep.world
        n = expert.numel()
        counts = torch.empty(n_experts, dtype=torch.int32, device=expert.device)
        self.slot = torch.empty(n, dtype=torch.int32, device=expert.device)
        _lib.check(_lib.lib().pb_moe_slots(_lib.ptr(expert), _lib.ptr(counts), _lib.ptr(self.slot), _lib.c_int(n),
                                           _lib.c_int(n_experts), _lib.stream_ptr()), "pb_moe_slots")
        if ep.world > 1:
            allc = torch.empty(ep.world, n_experts, dtype=torch.int32, device=expert.device)
            dist.all_gather_into_tensor(allc, counts, group=ep.group)
        else:
            allc = counts.view(1, -1)
        c = allc.cpu().tolist()  # [src][expert]; the one host sync of the layer: buffer sizes depend on it
        W, E, epr = ep.world, n_experts, self.experts_per_rank
        totals = [sum(c[s][e] for s in range(W)) for e in range(E)]
        dst_base = [0] * E
        for d in range(W):
            start = 0
            for e in range(d * epr, (d + 1) * epr):
                dst_base[e] = start + sum(c[s][e] for s in range(ep.rank))
                start += totals[e]
        self.dst_base = torch.tensor(dst_base, dtype=torch.int32, device=expert.device)
        mine = range(ep.rank * epr, (ep.rank + 1) * epr)
        self.local_totals: List[int] = [totals[e] for e in mine]
        self.recv_total = sum(self.local_totals)
        if self.recv_total > ep.capacity:
            raise RuntimeError(f"MoE receive buffer too small: {self.recv_total} rows > capacity {ep.capacity}")


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan: _Plan):
        ep = plan.ep
        ep.dispatch(x.contiguous(), plan.expert, plan.slot, plan.dst_base, None, plan.experts_per_rank)
        ctx.plan = plan
        ctx.T = x.shape[0]
        return ep.recv_rows(plan.recv_total).clone()

    @staticmethod
    def backward(ctx, d_recv):
        plan, ep = ctx.plan, ctx.plan.ep
        ep.y_rows(plan.recv_total).copy_(d_recv)
        dx = torch.empty(ctx.T, ep.hidden, dtype=torch.bfloat16, device=d_recv.device)
        ep.combine(dx, plan.expert, plan.slot, plan.dst_base, None, None, plan.experts_per_rank)
        return dx, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_local, weight, plan: _Plan, T: int):
        ep = plan.ep
        ep.y_rows(plan.recv_total).copy_(y_local)
        out = torch.empty(T, ep.hidden, dtype=torch.bfloat16, device=y_local.device)
        save = torch.empty(T * ep.top_k, ep.hidden, dtype=torch.bfloat16, device=y_local.device)
        w = weight.reshape(-1).float().contiguous()
        ep.combine(out, plan.expert, plan.slot, plan.dst_base, w, save, plan.experts_per_rank)
        ctx.save_for_backward(save, w)
        ctx.plan = plan
        ctx.wshape = weight.shape
        ctx.wdtype = weight.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        save, w = ctx.saved_tensors
        plan, ep = ctx.plan, ctx.plan.ep
        dout = dout.contiguous()
        T = dout.shape[0]
        dots = torch.empty(T * ep.top_k, dtype=torch.float32, device=dout.device)
        _lib.check(_lib.lib().pb_moe_rowdot(_lib.ptr(dout), _lib.ptr(save), _lib.ptr(dots), _lib.c_int(T),
                                            _lib.c_int(ep.top_k), _lib.c_int(ep.hidden), _lib.stream_ptr()),
                   "pb_moe_rowdot")
        ep.dispatch(dout, plan.expert, plan.slot, plan.dst_base, w, plan.experts_per_rank)
        dy_local = ep.recv_rows(plan.recv_total).clone()
        return dy_local, dots.view(ctx.wshape).to(ctx.wdtype), None, None


class _AuxLossInject(torch.autograd.Function):
    """Passes activations through and, in backward, feeds a gradient of 1 into ``aux`` (already multiplied by its
    coefficient): the load-balance loss of a middle pipeline stage reaches its router without travelling to the
    last stage."""

    @staticmethod
    def forward(ctx, x, aux):
        ctx.save_for_backward(aux)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        (aux,) = ctx.saved_tensors
        return g, torch.ones_like(aux)


class MoEFeedForward(nn.Module):
    """Top-k routed SwiGLU experts. ``n_experts`` in total, this rank holds ``n_experts / ep_size`` of them
    (expert ``e`` lives on rank ``e // experts_per_rank``). Input/output: ``[T, dim]``."""

    def __init__(self, dim: int, ffn_dim: int, n_experts: int, top_k: int = 2, ep: Optional[EPContext] = None,
                 ep_size: int = 1, ep_rank: int = 0, aux_coef: float = 0.01, init_std: float = 0.02, device=None,
                 dtype=None):
        super().__init__()
        assert n_experts % ep_size == 0
        self.dim, self.ffn_dim, self.n_experts, self.top_k = dim, ffn_dim, n_experts, top_k
        self.ep, self.ep_size, self.ep_rank, self.aux_coef = ep, ep_size, ep_rank, aux_coef
        self.local_experts = list(range(ep_rank * (n_experts // ep_size), (ep_rank + 1) * (n_experts // ep_size)))
        # the router GEMM needs a 16-byte row pitch on its output: rows beyond n_experts are padding (zero, unused)
        e_pad = (n_experts + 7) // 8 * 8
        self.router = nn.Parameter(torch.zeros(e_pad, dim, device=device, dtype=dtype))
        with torch.no_grad():
            self.router[:n_experts].normal_(std=init_std)
        self.w_gate_up = nn.ParameterDict()
        self.w_down = nn.ParameterDict()
        for e in self.local_experts:
            gu = nn.Parameter(torch.empty(2 * ffn_dim, dim, device=device, dtype=dtype))
            dn = nn.Parameter(torch.empty(dim, ffn_dim, device=device, dtype=dtype))
            nn.init.normal_(gu, std=init_std)
            nn.init.normal_(dn, std=init_std)
            self.w_gate_up[str(e)] = gu
            self.w_down[str(e)] = dn
        self.last_aux_loss: Optional[torch.Tensor] = None

    def _route(self, x):
        logits = pf.linear(x, self.router)[:, : self.n_experts].float()
        probs = logits.softmax(-1)
        topw, topi = probs.topk(self.top_k, dim=-1)
        topw = topw / topw.sum(-1, keepdim=True)
        # load-balance loss: E * sum_e (share of assignments to e) * (mean router probability of e)
        share = torch.zeros(self.n_experts, device=x.device, dtype=torch.float32)
        share.scatter_add_(0, topi.reshape(-1), torch.ones(topi.numel(), device=x.device))
        share = share / topi.numel()
        aux = self.n_experts * (share * probs.mean(0)).sum()
        return topw, topi, aux

    def forward(self, x):
        T = x.shape[0]
        topw, topi, aux = self._route(x)
        self.last_aux_loss = aux.detach()
        if self.aux_coef:
            x = _AuxLossInject.apply(x, aux * self.aux_coef)
        if self.ep is not None and x.is_cuda and x.dtype == torch.bfloat16:
            plan = _Plan(self.ep, topi.reshape(-1).to(torch.int32).contiguous(), self.n_experts)
            rows = _DispatchFn.apply(x, plan)
            outs, start = [], 0
            for e, n in zip(self.local_experts, plan.local_totals):
                xe = rows[start : start + n]
                start += n
                if n == 0:
                    outs.append(xe)
                    continue
                h = pf.swiglu(pf.linear(xe, self.w_gate_up[str(e)]))
                outs.append(pf.linear(h, self.w_down[str(e)]))
            y_local = torch.cat(outs, 0) if len(outs) > 1 else outs[0]
            return _CombineFn.apply(y_local, topw.to(x.dtype), plan, T)
        # dense reference path (one rank holds every expert): plain PyTorch statement of the same layer
        if self.ep_size != 1:
            raise RuntimeError("the reference MoE path needs all experts on one rank")
        out = torch.zeros_like(x, dtype=torch.float32)
        for e in self.local_experts:
            mask = topi == e
            tok = mask.any(-1).nonzero(as_tuple=True)[0]
            if tok.numel() == 0:
                continue
            w = (topw * mask).sum(-1)[tok]
            h = pf.swiglu(pf.linear(x[tok], self.w_gate_up[str(e)]))
            y = pf.linear(h, self.w_down[str(e)])
            out.index_add_(0, tok, y.float() * w[:, None].float())
        return out.to(x.dtype)
