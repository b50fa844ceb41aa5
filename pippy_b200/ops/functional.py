"""Differentiable ops of the package.

CUDA bf16 tensors run the hand-written sm_100a kernels (``csrc/``) through ctypes; anything else (CPU tensors,
fp32) takes a plain PyTorch implementation of the same math, which is also what the numerics tests compare the
kernels against.  There is no eager fallback for CUDA bf16: a missing library raises.

Parameter gradients of these ops are written by the ops themselves (into ``param.main_grad`` when the parameter
has one, an fp32 accumulation buffer, else into ``param.grad``) rather than returned to autograd.  That lets the
weight-gradient GEMM accumulate in fp32 in its epilogue and lets zero-bubble schedules postpone it: while a
:class:`pippy_b200.backward.defer_weight_grads` context is active the weight-gradient work is queued instead of
run.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from ..backward import current_deferral
from . import _lib
from .gemm import ACT_GELU_TANH, ACT_NONE, gemm


def _use_kernels(*tensors: torch.Tensor) -> bool:
    t = tensors[0]
    return t.is_cuda and t.dtype == torch.bfloat16


_SM_COUNT = {}


def sm_count() -> int:
    dev = torch.cuda.current_device()
    n = _SM_COUNT.get(dev)
    if n is None:
        n = torch.cuda.get_device_properties(dev).multi_processor_count
        _SM_COUNT[dev] = n
    return n


# ------------------------------------------------------------------------------------------------
# parameter-gradient plumbing
# ------------------------------------------------------------------------------------------------
def _accumulate_param_grad(param: torch.Tensor, grad: torch.Tensor) -> None:
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        if grad.dtype == torch.bfloat16 and mg.dtype == torch.float32 and grad.is_cuda and grad.numel() % 8 == 0:
            _lib.check(
                _lib.lib().pb_accum_bf16_into_f32(_lib.ptr(mg), _lib.ptr(grad.contiguous()), _lib.c_ll(grad.numel()),
                                                  _lib.stream_ptr()),
                "pb_accum_bf16_into_f32",
            )
        else:
            mg.add_(grad.to(mg.dtype).view_as(mg))
    elif param.grad is None:
        param.grad = grad.to(param.dtype).view_as(param).clone()
    else:
        param.grad.add_(grad.to(param.dtype).view_as(param))


def _run_or_defer(fn) -> None:
    q = current_deferral()
    if q is not None:
        q.defer(fn)
    else:
        fn()


# ------------------------------------------------------------------------------------------------
# linear
# ------------------------------------------------------------------------------------------------
def _wgrad(dy2: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> None:
    mg = getattr(weight, "main_grad", None)
    if mg is not None and mg.dtype == torch.float32:
        gemm(dy2, x2, a_mn=True, b_mn=True, out=mg.view(weight.shape), accumulate=True)
    else:
        dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        _accumulate_param_grad(weight, dw)
    if bias is not None and bias.requires_grad:
        bmg = getattr(bias, "main_grad", None)
        if bmg is not None and bmg.dtype == torch.float32:
            target = bmg
        else:
            target = torch.zeros(bias.shape, dtype=torch.float32, device=bias.device)
        _lib.check(
            _lib.lib().pb_colsum_bf16(_lib.ptr(dy2), _lib.ptr(target), _lib.c_ll(dy2.shape[0]),
                                      _lib.c_int(dy2.shape[1]), _lib.c_ll(dy2.stride(0)), _lib.stream_ptr()),
            "pb_colsum_bf16",
        )
        if target is not bmg:
            _accumulate_param_grad(bias, target)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual, act: int):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, residual.shape[-1])
            if not res2.is_contiguous():
                res2 = res2.contiguous()
        aux = None
        if act == ACT_GELU_TANH and (x.requires_grad or weight.requires_grad):
            aux = torch.empty(x2.shape[0], weight.shape[0], device=x.device, dtype=torch.bfloat16)
        y = gemm(x2, weight, bias=bias, residual=res2, act=act, aux=aux)
        weight._pb_direct_grad = True
        if bias is not None:
            bias._pb_direct_grad = True
        # Parameters ride on ctx, not in save_for_backward: saved tensors pass through the saved-tensor hooks of
        # activation checkpointing, which hand the backward a detached stand-in without `main_grad` or
        # `requires_grad`, and the weight gradient would be written to an object nobody reads.
        ctx.save_for_backward(x2, aux)
        ctx.weight = weight
        ctx.bias = bias
        ctx.act = act
        ctx.has_residual = residual is not None
        ctx.res_shape = residual.shape if residual is not None else None
        ctx.x_shape = x.shape
        # 2-D in, 2-D out: the result is returned as allocated, never as a view made in here (autograd refuses
        # in-place changes, such as the rotary embedding of a qkv projection, to views created inside a Function)
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, aux = ctx.saved_tensors
        weight, bias = ctx.weight, ctx.bias
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = dy.reshape(ctx.res_shape) if ctx.has_residual else None
        if ctx.act == ACT_GELU_TANH:
            dpre = torch.empty_like(dy2)
            _lib.check(
                _lib.lib().pb_gelu_bwd(_lib.ptr(dy2), _lib.ptr(aux), _lib.ptr(dpre), _lib.c_ll(dy2.numel()),
                                       _lib.stream_ptr()),
                "pb_gelu_bwd",
            )
            dy2 = dpre
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        if weight.requires_grad:
            _run_or_defer(lambda: _wgrad(dy2, x2, weight, bias))
        return dx, None, None, dres, None


def linear(x, weight, bias=None, residual=None, activation: Optional[str] = None):
    """``act(x @ weight.T + bias) + residual`` with everything after the GEMM fused into its epilogue."""
    if _use_kernels(x):
        act = ACT_GELU_TANH if activation == "gelu_tanh" else ACT_NONE
        if activation not in (None, "gelu_tanh"):
            raise ValueError(f"unsupported fused activation {activation!r}")
        y = _LinearFn.apply(x, weight, bias, residual, act)
        return y if x.dim() == 2 else y.view(*x.shape[:-1], weight.shape[0])
    y = F.linear(x, weight, bias)
    if activation == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    elif activation is not None:
        raise ValueError(f"unsupported fused activation {activation!r}")
    if residual is not None:
        y = y + residual
    return y


# ------------------------------------------------------------------------------------------------
# normalisation
# ------------------------------------------------------------------------------------------------
_NORM_SCRATCH = {}


def _norm_scratch(H: int, device) -> torch.Tensor:
    key = (device.index, H)
    buf = _NORM_SCRATCH.get(key)
    if buf is None:
        n = int(_lib.lib().pb_norm_bwd_scratch_floats(_lib.c_int(H), _lib.c_int(sm_count())))
        buf = torch.empty(n, dtype=torch.float32, device=device)
        _NORM_SCRATCH[key] = buf
    return buf


_lib_scratch_restype_set = False


def _ensure_restypes():
    global _lib_scratch_restype_set
    if not _lib_scratch_restype_set:
        _lib.lib().pb_norm_bwd_scratch_floats.restype = _lib.c_ll
        _lib_scratch_restype_set = True


class _NormFn(torch.autograd.Function):
    """``fork=True`` also returns the input itself as a second output: the caller feeds THAT to the residual
    branch, so both gradients of the tensor arrive here and the backward kernel adds the residual one to dx
    (autograd would otherwise sum them with an elementwise kernel of its own)."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps: float, layer: bool, fork: bool):
        _ensure_restypes()
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        mean = torch.empty(T, dtype=torch.float32, device=x.device) if layer else None
        _lib.check(
            _lib.lib().pb_norm_fwd(_lib.ptr(x2), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(y), _lib.ptr(mean),
                                   _lib.ptr(rstd), _lib.c_int(T), _lib.c_int(H), _lib.c_float(eps),
                                   _lib.c_int(int(layer)), _lib.stream_ptr()),
            "pb_norm_fwd",
        )
        ctx.save_for_backward(x2, mean, rstd)
        ctx.weight = weight  # not a saved tensor: see _LinearFn.forward
        weight._pb_direct_grad = True
        if bias is not None:
            bias._pb_direct_grad = True
        ctx.bias = bias
        ctx.layer = layer
        ctx.x_shape = x.shape
        ctx.set_materialize_grads(False)  # an unused branch of the fork arrives as None, not as a tensor of zeros
        if fork:
            return y.view(x.shape), x
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dres=None):
        x2, mean, rstd = ctx.saved_tensors
        weight, bias = ctx.weight, ctx.bias
        T, H = x2.shape
        if dy is None:  # only the residual branch was used
            return dres, None, None, None, None, None
        dy2 = dy.reshape(T, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if dres is not None:
            dres = dres.reshape(T, H)
            if dres.dtype != x2.dtype:
                dres = dres.to(x2.dtype)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        dx = torch.empty_like(x2)
        wmg = getattr(weight, "main_grad", None)
        use_main = wmg is not None and wmg.dtype == torch.float32
        dw = wmg if use_main else torch.empty(H, dtype=torch.float32, device=x2.device)
        db = None
        if ctx.layer:
            bmg = getattr(bias, "main_grad", None)
            db = bmg if (use_main and bmg is not None) else torch.empty(H, dtype=torch.float32, device=x2.device)
        _lib.check(
            _lib.lib().pb_norm_bwd_res(_lib.ptr(dy2), _lib.ptr(x2), _lib.ptr(weight), _lib.ptr(mean), _lib.ptr(rstd),
                                       _lib.ptr(dres), _lib.ptr(dx), _lib.ptr(dw), _lib.ptr(db), _lib.ptr(None),
                                       _lib.ptr(None), _lib.c_int(int(use_main)),
                                       _lib.ptr(_norm_scratch(H, x2.device)), _lib.c_int(T), _lib.c_int(H),
                                       _lib.c_int(int(ctx.layer)), _lib.c_int(sm_count()), _lib.stream_ptr()),
            "pb_norm_bwd_res",
        )
        if not use_main:
            _accumulate_param_grad(weight, dw)
            if ctx.layer:
                _accumulate_param_grad(bias, db)
        return dx.view(ctx.x_shape), None, None, None, None, None


def rms_norm_fork(x, weight, eps: float = 1e-5):
    """``(rms_norm(x), x)`` for the pre-norm residual pattern ``x + f(norm(x))``: use the second result as the
    residual operand.  On the kernel path the gradient that comes back through it is added to the norm's input
    gradient inside the norm-backward kernel."""
    if _use_kernels(x):
        return _NormFn.apply(x, weight, None, eps, False, True)
    return rms_norm(x, weight, eps), x


def rms_norm(x, weight, eps: float = 1e-5):
    if _use_kernels(x):
        return _NormFn.apply(x, weight, None, eps, False, False)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


def layer_norm(x, weight, bias, eps: float = 1e-5):
    if _use_kernels(x):
        return _NormFn.apply(x, weight, bias, eps, True, False)
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


# ------------------------------------------------------------------------------------------------
# activations
# ------------------------------------------------------------------------------------------------
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, row_limit=None):
        F2 = gu.shape[-1]
        g2 = gu.reshape(-1, F2)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        out = torch.empty(g2.shape[0], F2 // 2, device=gu.device, dtype=gu.dtype)
        _lib.check(
            _lib.lib().pb_swiglu_fwd(_lib.ptr(g2), _lib.ptr(out), _lib.c_ll(g2.shape[0]), _lib.c_int(F2 // 2),
                                     _lib.ptr(row_limit), _lib.stream_ptr()),
            "pb_swiglu_fwd",
        )
        ctx.save_for_backward(g2)
        ctx.row_limit = row_limit
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], F2 // 2)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        d2 = dout.reshape(g2.shape[0], -1)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dgu = torch.empty_like(g2)
        _lib.check(
            _lib.lib().pb_swiglu_bwd(_lib.ptr(d2), _lib.ptr(g2), _lib.ptr(dgu), _lib.c_ll(g2.shape[0]),
                                     _lib.c_int(g2.shape[1] // 2), _lib.ptr(ctx.row_limit), _lib.stream_ptr()),
            "pb_swiglu_bwd",
        )
        return dgu.view(ctx.shape), None


def swiglu(gate_up, row_limit=None):
    """``silu(gate) * up`` for ``gate_up = [..., gate | up]`` (two equal halves on the last dim).  ``row_limit``
    (an int32 device scalar, kernel path only) restricts the work to the first ``row_limit`` rows of a buffer that
    is sized for a capacity; the other rows of the result (and of the gradient) are left as allocated."""
    if _use_kernels(gate_up):
        return _SwiGLUFn.apply(gate_up, row_limit)
    g, u = gate_up.chunk(2, dim=-1)
    return F.silu(g) * u


# ------------------------------------------------------------------------------------------------
# RoPE + attention
# ------------------------------------------------------------------------------------------------
def rope_tables(seq_len: int, head_dim: int, theta: float, device) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32, device=device), inv)
    return ang.cos().contiguous(), ang.sin().contiguous()


def _rope_inplace(buf: torch.Tensor, cos, sin, T: int, S: int, n_heads: int, D: int, sign: float) -> None:
    _lib.check(
        _lib.lib().pb_rope(_lib.ptr(buf), _lib.ptr(cos), _lib.ptr(sin), _lib.c_ll(T), _lib.c_int(S),
                           _lib.c_int(n_heads), _lib.c_int(D), _lib.c_ll(buf.stride(0)), _lib.c_float(sign),
                           _lib.stream_ptr()),
        "pb_rope",
    )


def _rope_ref(x, cos, sin):  # x: [B, S, H, D]
    d2 = x.shape[-1] // 2
    a, b = x[..., :d2].float(), x[..., d2:].float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)


def flash_forward(q, k, v, B, S, Hq, Hkv, D, scale, causal=True):
    """Raw kernel call: q/k/v are 2-D views [B*S, heads*D] (unit inner stride); returns (o [B*S, Hq*D], lse)."""
    o = torch.empty(B * S, Hq * D, device=q.device, dtype=torch.bfloat16)
    lse = torch.empty(B, Hq, S, device=q.device, dtype=torch.float32)
    _lib.check(
        _lib.lib().pb_flash_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.c_int(B),
                                _lib.c_int(S), _lib.c_int(Hq), _lib.c_int(Hkv), _lib.c_int(D),
                                _lib.c_ll(q.stride(0)), _lib.c_ll(k.stride(0)), _lib.c_ll(v.stride(0)),
                                _lib.c_ll(o.stride(0)), _lib.c_float(scale), _lib.c_int(int(causal)),
                                _lib.ptr(_lib.err_word(q.device)), _lib.stream_ptr()),
        "pb_flash_fwd",
    )
    return o, lse


def flash_backward(do, q, k, v, o, lse, B, S, Hq, Hkv, D, scale, causal=True, dqkv: Optional[torch.Tensor] = None):
    """Raw kernel call: returns (dq, dk, dv) as views into one packed [B*S, (Hq + 2 Hkv) * D] buffer."""
    T = B * S
    if dqkv is None:
        dqkv = torch.empty(T, (Hq + 2 * Hkv) * D, device=q.device, dtype=torch.bfloat16)
    dq = dqkv[:, : Hq * D]
    dk = dqkv[:, Hq * D : (Hq + Hkv) * D]
    dv = dqkv[:, (Hq + Hkv) * D :]
    delta = torch.empty(B, Hq, S, device=q.device, dtype=torch.float32)
    _lib.check(
        _lib.lib().pb_flash_bwd(_lib.ptr(do), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse),
                                _lib.ptr(delta), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.c_int(B),
                                _lib.c_int(S), _lib.c_int(Hq), _lib.c_int(Hkv), _lib.c_int(D),
                                _lib.c_ll(q.stride(0)), _lib.c_ll(k.stride(0)), _lib.c_ll(v.stride(0)),
                                _lib.c_ll(o.stride(0)), _lib.c_ll(do.stride(0)), _lib.c_ll(dqkv.stride(0)),
                                _lib.c_float(scale), _lib.c_int(int(causal)), _lib.ptr(_lib.err_word(q.device)),
                                _lib.stream_ptr()),
        "pb_flash_bwd",
    )
    return dq, dk, dv, dqkv


class _RopeAttentionFn(torch.autograd.Function):
    """qkv [B*S, (Hq + 2 Hkv) * D] -> attention output [B*S, Hq * D].

    RoPE is applied to the q and k columns of ``qkv`` IN PLACE (the rotated projection is what the backward needs,
    and a second copy of the largest activation of the layer would be kept for nothing).  The kernel writes through
    a raw pointer, so the tensor's version counter is bumped by hand: a producer that had saved ``qkv`` for its own
    backward gets autograd's usual "modified by an inplace operation" error instead of silently wrong gradients.
    The gradient returned for ``qkv`` is with respect to its value BEFORE the rotation."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, B, S, Hq, Hkv, D, scale, causal):
        T = B * S
        if cos is not None:
            _rope_inplace(qkv, cos, sin, T, S, Hq + Hkv, D, 1.0)
            torch.autograd.graph.increment_version(qkv)
        q = qkv[:, : Hq * D]
        k = qkv[:, Hq * D : (Hq + Hkv) * D]
        v = qkv[:, (Hq + Hkv) * D :]
        o, lse = flash_forward(q, k, v, B, S, Hq, Hkv, D, scale, causal)
        ctx.save_for_backward(qkv, o, lse, cos, sin)
        ctx.cfg = (B, S, Hq, Hkv, D, scale, causal)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, cos, sin = ctx.saved_tensors
        B, S, Hq, Hkv, D, scale, causal = ctx.cfg
        q = qkv[:, : Hq * D]
        k = qkv[:, Hq * D : (Hq + Hkv) * D]
        v = qkv[:, (Hq + Hkv) * D :]
        if not do.is_contiguous():
            do = do.contiguous()
        _, _, _, dqkv = flash_backward(do, q, k, v, o, lse, B, S, Hq, Hkv, D, scale, causal)
        if cos is not None:
            _rope_inplace(dqkv, cos, sin, B * S, S, Hq + Hkv, D, -1.0)
        return dqkv, None, None, None, None, None, None, None, None, None


def rope_attention(qkv, cos, sin, B: int, S: int, Hq: int, Hkv: int, D: int, scale: Optional[float] = None,
                   causal: bool = True):
    """Causal self-attention over a packed projection ``qkv`` of shape ``[B*S, (Hq + 2*Hkv) * D]``
    (q heads, then k heads, then v heads), with rotary embedding of q and k when ``cos``/``sin`` are given.

    On the kernel path (CUDA bf16) the rotation overwrites the q and k columns of ``qkv``: the caller's tensor holds
    the rotated projection afterwards (its version counter is bumped).  Pass a clone to keep the original.  The
    CPU path leaves ``qkv`` untouched."""
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    if _use_kernels(qkv):
        return _RopeAttentionFn.apply(qkv, cos, sin, B, S, Hq, Hkv, D, scale, causal)
    q = qkv[:, : Hq * D].view(B, S, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hkv) * D].view(B, S, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D :].view(B, S, Hkv, D)
    if cos is not None:
        q, k = _rope_ref(q, cos, sin), _rope_ref(k, cos, sin)
    rep = Hq // Hkv
    k = k.repeat_interleave(rep, dim=2)
    v = v.repeat_interleave(rep, dim=2)
    att = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril()
        att = att.masked_fill(~mask, float("-inf"))
    att = att.softmax(-1)
    out = torch.einsum("bhqk,bkhd->bqhd", att, v.float()).to(qkv.dtype)
    return out.reshape(B * S, Hq * D)


# ------------------------------------------------------------------------------------------------
# cross entropy
# ------------------------------------------------------------------------------------------------
class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, vocab: int, reduction: str, ignore_index: int, inplace: bool):
        T, ld = logits.shape
        tgt = targets.reshape(-1).contiguous()
        loss_rows = torch.empty(T, dtype=torch.float32, device=logits.device)
        dlogits = logits if inplace else torch.empty_like(logits)
        if reduction == "mean":
            n_valid = (tgt != ignore_index).sum().clamp(min=1).to(torch.float32)
        else:
            n_valid = None
        _lib.check(
            _lib.lib().pb_xent_fwd_bwd(_lib.ptr(logits), _lib.ptr(dlogits), _lib.ptr(tgt), _lib.ptr(loss_rows),
                                       _lib.c_ll(T), _lib.c_int(vocab), _lib.c_ll(logits.stride(0)),
                                       _lib.c_float(1.0), _lib.c_ll(ignore_index), _lib.stream_ptr()),
            "pb_xent_fwd_bwd",
        )
        loss = loss_rows.sum()
        if n_valid is not None:
            loss = loss / n_valid
        ctx.save_for_backward(dlogits, n_valid)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        dlogits, n_valid = ctx.saved_tensors
        scale = dloss.to(torch.float32).reshape(1)
        if n_valid is not None:
            scale = scale / n_valid
        scale = scale.contiguous()
        _lib.check(
            _lib.lib().pb_scale_bf16(_lib.ptr(dlogits), _lib.ptr(scale), _lib.c_ll(dlogits.numel()),
                                     _lib.stream_ptr()),
            "pb_scale_bf16",
        )
        return dlogits, None, None, None, None, None


def cross_entropy(logits, targets, vocab_size: Optional[int] = None, reduction: str = "mean",
                  ignore_index: int = -100, inplace: bool = False):
    """Softmax cross-entropy over ``logits [T, V_padded]``; columns at or beyond ``vocab_size`` are padding.
    With ``inplace=True`` the gradient overwrites ``logits`` (saves one [T, V] buffer)."""
    if reduction not in ("mean", "sum"):
        raise ValueError("reduction must be 'mean' or 'sum'")
    logits2 = logits.reshape(-1, logits.shape[-1])
    V = logits2.shape[-1] if vocab_size is None else vocab_size
    if _use_kernels(logits2):
        if not logits2.is_contiguous():
            logits2 = logits2.contiguous()
        return _CrossEntropyFn.apply(logits2, targets, V, reduction, ignore_index, inplace)
    return F.cross_entropy(logits2[:, :V].float(), targets.reshape(-1), reduction=reduction, ignore_index=ignore_index)


# ------------------------------------------------------------------------------------------------
# embedding
# ------------------------------------------------------------------------------------------------
def _embed_wgrad(ids, dout, wte, wpe, S):
    T, H = dout.shape
    wmg = getattr(wte, "main_grad", None)
    dw = wmg if (wmg is not None and wmg.dtype == torch.float32) else torch.zeros(wte.shape, dtype=torch.float32, device=wte.device)
    dp = None
    if wpe is not None:
        pmg = getattr(wpe, "main_grad", None)
        dp = pmg if (pmg is not None and pmg.dtype == torch.float32) else torch.zeros(wpe.shape, dtype=torch.float32, device=wpe.device)
    _lib.check(
        _lib.lib().pb_embed_bwd(_lib.ptr(ids), _lib.ptr(dout), _lib.ptr(dw), _lib.ptr(dp), _lib.c_ll(T),
                                _lib.c_int(H), _lib.c_int(S), _lib.c_ll(wte.shape[0]), _lib.stream_ptr()),
        "pb_embed_bwd",
    )
    if dw is not wmg:
        _accumulate_param_grad(wte, dw)
    if wpe is not None and dp is not getattr(wpe, "main_grad", None):
        _accumulate_param_grad(wpe, dp)


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, wte, wpe, S: int):
        flat = ids.reshape(-1).contiguous()
        T, H = flat.numel(), wte.shape[1]
        out = torch.empty(T, H, device=wte.device, dtype=wte.dtype)
        _lib.check(
            _lib.lib().pb_embed_fwd(_lib.ptr(flat), _lib.ptr(wte), _lib.ptr(wpe), _lib.ptr(out), _lib.c_ll(T),
                                    _lib.c_int(H), _lib.c_int(S), _lib.c_ll(wte.shape[0]), _lib.stream_ptr()),
            "pb_embed_fwd",
        )
        ctx.save_for_backward(flat)
        wte._pb_direct_grad = True
        if wpe is not None:
            wpe._pb_direct_grad = True
        ctx.params = (wte, wpe)
        ctx.S = S
        return out

    @staticmethod
    def backward(ctx, dout):
        (flat,) = ctx.saved_tensors
        wte, wpe = ctx.params
        d2 = dout.contiguous()
        S = ctx.S
        _run_or_defer(lambda: _embed_wgrad(flat, d2, wte, wpe, S))
        return None, None, None, None


def embedding(ids, wte, wpe=None, seq_len: Optional[int] = None):
    """``wte[ids] (+ wpe[position])`` flattened to ``[B*S, H]``; position of token t is ``t % seq_len``."""
    S = ids.shape[-1] if seq_len is None else seq_len
    if wte.is_cuda and wte.dtype == torch.bfloat16:
        # autograd only tracks the op if some input requires grad; tie it to the table
        return _EmbeddingFn.apply(ids, wte, wpe, S)
    out = F.embedding(ids.reshape(-1), wte)
    if wpe is not None:
        pos = torch.arange(ids.numel(), device=ids.device) % S
        out = out + F.embedding(pos, wpe)
    return out
