"""Expert parallelism for sparse MoE layers (top-k routing, SwiGLU experts) on fused NVLink kernels.

Per MoE layer and microbatch, on every rank of the expert-parallel group, with no host synchronisation anywhere
(every size that depends on the routing stays in device memory):

  route      router GEMM (tcgen05), then ONE kernel pair: softmax, top-k, normalised weights, load-balance loss and
             the position of each assignment inside its expert's group (``csrc/moe.cu``)
  dispatch   ONE kernel: the ranks exchange their per-expert row counts through peer memory, derive the layout of
             every receive buffer from them, permute the token rows and store each straight into the receive buffer
             of the rank that owns the expert, grouped by expert (P2P stores, flag handshakes)
  experts    ONE grouped tcgen05 GEMM launch per projection over all local experts; the kernel reads the group
             table the dispatch left in device memory and runs only the tiles that hold rows (``csrc/gemm.cu``)
  combine    ONE kernel pulls every token's k expert rows back from the owning ranks, un-permutes and forms the
             weighted sum in fp32

Backward swaps the roles: the gradient of ``combine`` is a dispatch of ``w * dy`` rows (plus a row-dot kernel for
the router-weight gradients), the gradient of ``dispatch`` is a combine with unit weights, the expert weight
gradients are one grouped GEMM per projection whose contraction runs over each expert's rows.  Receive buffers have a
fixed capacity (``capacity_factor`` times the even share); a routing that would overflow it raises the device error
word (checked by ``ops._lib.check_device_errors``) instead of writing out of bounds.  The reference has no expert
parallelism; its MoE example places whole experts on pipeline stages
(examples/mixture_of_experts/dist_moe.py:43-59).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import _lib
from ..ops import functional as pf
from ..ops.functional import _run_or_defer


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class EPContext:
    """Peer-mapped workspaces of one expert-parallel group, shared by all MoE layers (calls are stream ordered).

    ``capacity`` rows fit into a rank's receive buffer: ``capacity_factor`` times the rows it gets when the routing is
    perfectly even (``max_tokens * top_k``), plus the padding that lets every expert's group start on a multiple of
    256 rows."""

    def __init__(self, group: Optional[dist.ProcessGroup], max_tokens: int, hidden: int, top_k: int = 2,
                 n_experts: int = 8, device=None, ctas: int = 96, capacity_factor: float = 2.0):
        from ..comm.symm import SymmetricBuffer

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.hidden, self.top_k, self.ctas, self.n_experts = hidden, top_k, ctas, n_experts
        if n_experts % self.world != 0:
            raise ValueError(f"{n_experts} experts cannot be spread evenly over {self.world} ranks")
        self.experts_per_rank = n_experts // self.world
        even = max_tokens * top_k
        self.capacity = _align(int(even * min(capacity_factor, float(self.world))), 256) + 256 * self.experts_per_rank
        nbytes = self.capacity * hidden * 2
        self.recv = SymmetricBuffer(nbytes, group, self.device)
        self.ybuf = SymmetricBuffer(nbytes, group, self.device)
        self.cnt = SymmetricBuffer(self.world * n_experts * 4, group, self.device)
        self.flags_d = SymmetricBuffer(4096, group, self.device)
        self.flags_c = SymmetricBuffer(4096, group, self.device)
        self.counter = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.recv_ptrs = torch.tensor(self.recv.ptrs, dtype=torch.int64, device=self.device)
        self.y_ptrs = torch.tensor(self.ybuf.ptrs, dtype=torch.int64, device=self.device)
        self.cnt_ptrs = torch.tensor(self.cnt.ptrs, dtype=torch.int64, device=self.device)
        self.epoch_d = 0
        self.epoch_c = 0

    def _flags(self, buf):
        arr = (ctypes.POINTER(ctypes.c_int) * self.world)()
        for i, ptr in enumerate(buf.ptrs):
            arr[i] = ctypes.cast(ctypes.c_void_p(ptr), ctypes.POINTER(ctypes.c_int))
        return arr

    def recv_rows(self) -> torch.Tensor:
        return self.recv.tensor(torch.bfloat16, self.capacity * self.hidden).view(self.capacity, self.hidden)

    def y_rows(self) -> torch.Tensor:
        return self.ybuf.tensor(torch.bfloat16, self.capacity * self.hidden).view(self.capacity, self.hidden)

    def dispatch(self, x, plan: "_Plan", scale) -> None:
        T = x.shape[0]
        self.epoch_d += 1
        rc = _lib.lib().pb_moe_dispatch(
            _lib.ptr(x), _lib.ptr(plan.expert), _lib.ptr(plan.slot), _lib.ptr(plan.counts), _lib.ptr(scale),
            _lib.ptr(self.recv_ptrs), _lib.ptr(self.cnt_ptrs), _lib.c_int(T), _lib.c_int(self.top_k),
            _lib.c_int(self.hidden), _lib.c_int(self.n_experts), _lib.c_int(self.experts_per_rank),
            _lib.c_int(self.capacity), _lib.ptr(plan.dst_base), _lib.ptr(plan.group_rows),
            _lib.ptr(plan.group_start), _lib.ptr(plan.rows_used), self._flags(self.flags_d), _lib.ptr(self.counter),
            _lib.ptr(_lib.err_word(x.device)), _lib.c_int(self.rank), _lib.c_int(self.world),
            _lib.c_int(self.epoch_d), _lib.c_int(self.ctas), _lib.stream_ptr())
        _lib.check(rc, "pb_moe_dispatch")

    def combine(self, out, plan: "_Plan", weight, save) -> None:
        T = out.shape[0]
        self.epoch_c += 1
        rc = _lib.lib().pb_moe_combine(
            _lib.ptr(out), _lib.ptr(plan.expert), _lib.ptr(plan.slot), _lib.ptr(plan.dst_base), _lib.ptr(weight),
            _lib.ptr(self.y_ptrs), _lib.ptr(save), _lib.c_int(T), _lib.c_int(self.top_k), _lib.c_int(self.hidden),
            _lib.c_int(self.experts_per_rank), _lib.c_int(self.capacity), self._flags(self.flags_c),
            _lib.ptr(self.counter[1:]),
            _lib.ptr(_lib.err_word(out.device)), _lib.c_int(self.rank), _lib.c_int(self.world),
            _lib.c_int(self.epoch_c), _lib.c_int(self.ctas), _lib.stream_ptr())
        _lib.check(rc, "pb_moe_combine")


class _Plan:
    """Routing result of one layer call, all in device memory, shared by the autograd nodes of the layer."""

    def __init__(self, ep: EPContext, T: int):
        dev = ep.device
        E, k = ep.n_experts, ep.top_k
        self.ep = ep
        self.T = T
        self.expert = torch.empty(T * k, dtype=torch.int32, device=dev)   # expert of assignment (t, j)
        self.slot = torch.empty(T * k, dtype=torch.int32, device=dev)     # its position among this rank's rows for that expert
        self.counts = torch.empty(E, dtype=torch.int32, device=dev)       # this rank's rows per expert
        self.share = torch.empty(E, dtype=torch.float32, device=dev)
        self.dst_base = torch.empty(E, dtype=torch.int32, device=dev)     # filled by the dispatch kernel
        self.group_rows = torch.zeros(ep.experts_per_rank, dtype=torch.int32, device=dev)
        self.group_start = torch.zeros(ep.experts_per_rank, dtype=torch.int32, device=dev)
        self.rows_used = torch.zeros(1, dtype=torch.int32, device=dev)  # rows that hold a group or its padding


class _RouteFn(torch.autograd.Function):
    """logits [T, E_pad] -> (normalised top-k weights [T, k] fp32, load-balance loss); indices, positions and counts
    go into ``plan``."""

    @staticmethod
    def forward(ctx, logits, plan: _Plan, E: int, k: int):
        T, ld = logits.shape
        dev = logits.device
        probs = torch.empty(T, E, dtype=torch.float32, device=dev)
        topw = torch.empty(T, k, dtype=torch.float32, device=dev)
        aux = torch.empty((), dtype=torch.float32, device=dev)
        n_cta = (T + 255) // 256
        scratch_i = torch.empty(n_cta * E, dtype=torch.int32, device=dev)
        scratch_f = torch.empty(n_cta * E, dtype=torch.float32, device=dev)
        _lib.check(_lib.lib().pb_moe_route(
            _lib.ptr(logits), _lib.c_int(ld), _lib.c_int(T), _lib.c_int(E), _lib.c_int(k), _lib.ptr(probs),
            _lib.ptr(plan.expert), _lib.ptr(topw), _lib.ptr(plan.slot), _lib.ptr(plan.counts), _lib.ptr(plan.share),
            _lib.ptr(aux), _lib.ptr(scratch_i), _lib.ptr(scratch_f), _lib.stream_ptr()), "pb_moe_route")
        ctx.save_for_backward(probs, topw)
        ctx.plan, ctx.dims = plan, (T, E, k, ld)
        return topw, aux

    @staticmethod
    def backward(ctx, g_w, g_aux):
        probs, topw = ctx.saved_tensors
        plan = ctx.plan
        T, E, k, ld = ctx.dims
        dlogits = torch.empty(T, ld, dtype=torch.bfloat16, device=probs.device)
        g_w = None if g_w is None else g_w.float().contiguous()
        g_aux = None if g_aux is None else g_aux.float().contiguous()
        _lib.check(_lib.lib().pb_moe_route_bwd(
            _lib.ptr(probs), _lib.ptr(plan.expert), _lib.ptr(topw), _lib.ptr(g_w), _lib.ptr(g_aux),
            _lib.ptr(plan.share), _lib.c_int(T), _lib.c_int(E), _lib.c_int(k), _lib.ptr(dlogits), _lib.c_int(ld),
            _lib.stream_ptr()), "pb_moe_route_bwd")
        return dlogits, None, None, None


def grouped_gemm(mode: int, a, b, out, n, k_dim, plan: _Plan, b_mn: bool = False, accumulate: bool = False):
    """Thin wrapper of ``pb_gemm_grouped``: ``mode`` 1 groups the rows of ``a`` / ``out``, 2 the contraction."""
    G = plan.ep.experts_per_rank
    M = a.shape[0] if mode == 1 else a.shape[1]
    rc = _lib.lib().pb_gemm_grouped(
        _lib.c_int(mode), _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.c_int(M), _lib.c_int(n), _lib.c_int(k_dim),
        _lib.c_ll(a.stride(0)), _lib.c_ll(b.stride(-2)), _lib.c_ll(out.stride(-2)), _lib.c_int(int(b_mn)),
        _lib.c_int(G), _lib.ptr(plan.group_rows), _lib.ptr(plan.group_start),
        _lib.c_int(int(out.dtype == torch.float32)), _lib.c_int(int(accumulate)),
        _lib.ptr(_lib.err_word(a.device)), _lib.stream_ptr())
    _lib.check(rc, "pb_gemm_grouped")
    return out


class _GroupedLinearFn(torch.autograd.Function):
    """``y[r] = a[r] @ weight[g].T`` for the rows r of local expert g; ``weight`` is ``[G, N, K]``."""

    @staticmethod
    def forward(ctx, a, weight, plan: _Plan):
        G, N, K = weight.shape
        out = torch.empty(a.shape[0], N, dtype=torch.bfloat16, device=a.device)
        grouped_gemm(1, a, weight, out, N, K, plan)
        ctx.save_for_backward(a)
        ctx.weight, ctx.plan = weight, plan  # the parameter rides on ctx (see ops.functional._LinearFn)
        weight._pb_direct_grad = True
        return out

    @staticmethod
    def backward(ctx, dy):
        (a,) = ctx.saved_tensors
        weight, plan = ctx.weight, ctx.plan
        G, N, K = weight.shape
        dy = dy.contiguous()
        da = None
        if ctx.needs_input_grad[0]:
            da = torch.empty_like(a)
            grouped_gemm(1, dy, weight, da, K, N, plan, b_mn=True)

        def wgrad():
            mg = getattr(weight, "main_grad", None)
            if mg is not None and mg.dtype == torch.float32:
                grouped_gemm(2, dy, a, mg, K, a.shape[0], plan, accumulate=True)
            else:
                dw = torch.empty(G, N, K, dtype=torch.bfloat16, device=a.device)
                grouped_gemm(2, dy, a, dw, K, a.shape[0], plan)
                pf._accumulate_param_grad(weight, dw)

        if weight.requires_grad:
            _run_or_defer(wgrad)
        return da, None, None


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan: _Plan):
        ep = plan.ep
        ep.dispatch(x.contiguous(), plan, None)
        ctx.plan = plan
        ctx.T = x.shape[0]
        # the receive buffer is shared by all layers: the rows are copied out (they are also what the expert
        # weight gradients need later)
        return ep.recv_rows().clone()

    @staticmethod
    def backward(ctx, d_recv):
        plan, ep = ctx.plan, ctx.plan.ep
        ep.y_rows().copy_(d_recv)  # into the peer-mapped buffer the owners of the tokens pull from
        dx = torch.empty(ctx.T, ep.hidden, dtype=torch.bfloat16, device=d_recv.device)
        ep.combine(dx, plan, None, None)
        return dx, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_local, weight, plan: _Plan, T: int):
        ep = plan.ep
        ep.y_rows().copy_(y_local)  # into the peer-mapped buffer the owners of the tokens pull from
        out = torch.empty(T, ep.hidden, dtype=torch.bfloat16, device=y_local.device)
        save = torch.empty(T * ep.top_k, ep.hidden, dtype=torch.bfloat16, device=y_local.device)
        w = weight.reshape(-1).float().contiguous()
        ep.combine(out, plan, w, save)
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
        ep.dispatch(dout, plan, w)
        dy_local = ep.recv_rows().clone()
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
    (expert ``e`` lives on rank ``e // experts_per_rank``) as two stacked parameters ``w_gate_up [local, 2 ffn, dim]``
    and ``w_down [local, dim, ffn]``. Input/output: ``[T, dim]``."""

    def __init__(self, dim: int, ffn_dim: int, n_experts: int, top_k: int = 2, ep: Optional[EPContext] = None,
                 ep_size: int = 1, ep_rank: int = 0, aux_coef: float = 0.01, init_std: float = 0.02, device=None,
                 dtype=None):
        super().__init__()
        assert n_experts % ep_size == 0
        self.dim, self.ffn_dim, self.n_experts, self.top_k = dim, ffn_dim, n_experts, top_k
        self.ep, self.ep_size, self.ep_rank, self.aux_coef = ep, ep_size, ep_rank, aux_coef
        n_local = n_experts // ep_size
        self.local_experts = list(range(ep_rank * n_local, (ep_rank + 1) * n_local))
        if ep is not None and (ep.n_experts != n_experts or ep.top_k != top_k or ep.hidden != dim):
            raise ValueError("the expert-parallel context was built for another layer shape")
        # the router GEMM needs a 16-byte row pitch on its output: rows beyond n_experts are padding (zero, unused)
        e_pad = (n_experts + 7) // 8 * 8
        self.router = nn.Parameter(torch.zeros(e_pad, dim, device=device, dtype=dtype))
        self.w_gate_up = nn.Parameter(torch.empty(n_local, 2 * ffn_dim, dim, device=device, dtype=dtype))
        self.w_down = nn.Parameter(torch.empty(n_local, dim, ffn_dim, device=device, dtype=dtype))
        with torch.no_grad():
            self.router[:n_experts].normal_(std=init_std)
            self.w_gate_up.normal_(std=init_std)
            self.w_down.normal_(std=init_std)
        self.last_aux_loss: Optional[torch.Tensor] = None

    def _route_reference(self, x):
        logits = F.linear(x, self.router)[:, : self.n_experts].float()
        probs = logits.softmax(-1)
        # a stable sort breaks ties towards the lower expert index, as the router kernel does
        order = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, : self.top_k]
        topi = order
        topw = probs.gather(-1, topi)
        topw = topw / topw.sum(-1, keepdim=True)
        # load-balance loss: E * sum_e (share of assignments to e) * (mean router probability of e)
        share = torch.zeros(self.n_experts, device=x.device, dtype=torch.float32)
        share.scatter_add_(0, topi.reshape(-1), torch.ones(topi.numel(), device=x.device))
        share = share / topi.numel()
        aux = self.n_experts * (share * probs.mean(0)).sum()
        return topw, topi, aux

    def forward(self, x):
        T = x.shape[0]
        if self.ep is not None and x.is_cuda and x.dtype == torch.bfloat16:
            plan = _Plan(self.ep, T)
            logits = pf.linear(x, self.router)
            topw, aux = _RouteFn.apply(logits, plan, self.n_experts, self.top_k)
            self.last_aux_loss = aux.detach()
            if self.aux_coef:
                x = _AuxLossInject.apply(x, aux * self.aux_coef)
            rows = _DispatchFn.apply(x, plan)
            h = pf.swiglu(_GroupedLinearFn.apply(rows, self.w_gate_up, plan), row_limit=plan.rows_used)
            y_local = _GroupedLinearFn.apply(h, self.w_down, plan)
            return _CombineFn.apply(y_local, topw, plan, T)
        # dense reference path (one rank holds every expert): plain PyTorch statement of the same layer
        if self.ep_size != 1:
            raise RuntimeError("the reference MoE path needs all experts on one rank")
        topw, topi, aux = self._route_reference(x)
        self.last_aux_loss = aux.detach()
        if self.aux_coef:
            x = _AuxLossInject.apply(x, aux * self.aux_coef)
        out = torch.zeros_like(x, dtype=torch.float32)
        for i, e in enumerate(self.local_experts):
            mask = topi == e
            tok = mask.any(-1).nonzero(as_tuple=True)[0]
            if tok.numel() == 0:
                continue
            w = (topw * mask).sum(-1)[tok]
            g, u = F.linear(x[tok], self.w_gate_up[i]).chunk(2, dim=-1)
            y = F.linear(F.silu(g) * u, self.w_down[i])
            out.index_add_(0, tok, y.float() * w[:, None].float())
        return out.to(x.dtype)
