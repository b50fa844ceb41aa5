"""Tensor parallelism with sequence-parallel activations, on fused compute+collective kernels.

Activations between the parallel regions are sharded along the token dimension (``[T / tp, d]``).  A column-parallel
linear starts with an all-gather of those shards and a row-parallel linear ends with a reduce-scatter; here each pair
is ONE kernel (``csrc/gemm.cu``, fused modes): copy CTAs pull the peers' shards over NVLink while the tcgen05 GEMM
already runs on the rows that have arrived, and the GEMM epilogue stores foreign output tiles straight into their
owner's memory before the grid sums what it received.  The reference has no tensor parallelism of its own; its
example composes with DTensor (examples/tp+pp/pippy_tp.py:79-112), i.e. NCCL all-gather / reduce-scatter around
cuBLAS GEMMs.

Backward duals: d(input) of a column-parallel linear is a GEMM -> reduce-scatter, d(input) of a row-parallel linear an
all-gather -> GEMM (whose gathered rows also feed that layer's weight gradient); the column-parallel weight gradient
re-gathers its input with the package's own peer-memory all-gather kernel and runs a local GEMM.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..comm.symm import SymmetricBuffer
from ..ops import _lib
from ..ops.functional import _accumulate_param_grad
from ..ops.gemm import gemm


class TPContext:
    """Peer-mapped workspaces of one tensor-parallel group, shared by all layers (calls are stream ordered).

    ``max_rows`` is the per-rank shard length (tokens / tp, a multiple of 256), ``max_cols`` the widest activation
    that is gathered or scattered."""

    def __init__(self, group: Optional[dist.ProcessGroup], max_rows: int, max_cols: int, device=None, copy_ctas: int = 8):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        if max_rows % 256 != 0:
            raise ValueError("the per-rank shard length must be a multiple of 256 tokens")
        self.max_rows, self.max_cols = max_rows, max_cols
        self.copy_ctas = copy_ctas
        W = self.world
        self.ag_src = SymmetricBuffer(max_rows * max_cols * 2, group, self.device)
        self.ag_flags = SymmetricBuffer(4096, group, self.device)
        self.rs_staging = SymmetricBuffer(W * max_rows * max_cols * 2, group, self.device)
        self.rs_flags = SymmetricBuffer(4096, group, self.device)
        self.gathered = torch.empty(W * max_rows * max_cols, dtype=torch.bfloat16, device=self.device)
        self.rs_scratch = torch.empty(max_rows * max_cols, dtype=torch.bfloat16, device=self.device)
        self.tile_flags = torch.zeros(W * max_rows // 256 + 8, dtype=torch.int32, device=self.device)
        self.counters = torch.zeros(16, dtype=torch.int32, device=self.device)
        self.gather_flags = SymmetricBuffer(4096, group, self.device)
        self.gather_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.ag_epoch = 0
        self.rs_epoch = 0
        self.gather_epoch = 0

    def _flag_array(self, buf: SymmetricBuffer):
        arr = (ctypes.POINTER(ctypes.c_int) * self.world)()
        for i, ptr in enumerate(buf.ptrs):
            arr[i] = ctypes.cast(ctypes.c_void_p(ptr), ctypes.POINTER(ctypes.c_int))
        return arr

    # ------------------------------------------------------------------ fused ops
    def ag_gemm(self, x_shard: torch.Tensor, weight: torch.Tensor, b_mn: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        """``concat_ranks(x_shard) @ weight.T`` (or ``@ weight`` when ``b_mn``). Returns ``(y, gathered_x)``;
        ``gathered_x`` is a view of the workspace, valid until the next ``ag_gemm``. Rows of this rank inside it are
        NOT filled (they are read from ``x_shard`` in place)."""
        rows, K = x_shard.shape
        N = weight.shape[1] if b_mn else weight.shape[0]
        W = self.world
        assert rows % 256 == 0 and rows <= self.max_rows and K <= self.max_cols
        src = self.ag_src.tensor(torch.bfloat16, rows * K).view(rows, K)
        src.copy_(x_shard)  # publish the shard where the peers can read it
        gathered = self.gathered[: W * rows * K].view(W * rows, K)
        y = torch.empty(W * rows, N, dtype=torch.bfloat16, device=x_shard.device)
        self.ag_epoch += 1
        rc = _lib.lib().pb_gemm_tp_fused(
            _lib.c_int(1), _lib.ptr(src), _lib.ptr(weight), _lib.ptr(y), _lib.c_int(N), _lib.c_int(K),
            _lib.c_ll(K), _lib.c_ll(weight.stride(0)), _lib.c_ll(N), _lib.c_int(int(b_mn)), _lib.c_int(self.rank),
            _lib.c_int(W), _lib.c_int(rows), _lib.c_int(self.ag_epoch), self.ag_src.pointer_array(),
            _lib.ptr(gathered), None, None, None, self._flag_array(self.ag_flags), _lib.ptr(self.tile_flags),
            _lib.ptr(self.counters), _lib.c_int(self.copy_ctas), _lib.ptr(_lib.err_word(x_shard.device)),
            _lib.stream_ptr(),
        )
        _lib.check(rc, "pb_gemm_tp_fused(all-gather -> GEMM)")
        return y, gathered

    def gemm_rs(self, x: torch.Tensor, weight: torch.Tensor, b_mn: bool = False,
                residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``reduce_scatter_rows(x @ weight.T)`` (+ ``residual`` on the local shard). ``x`` is ``[T, K_local]``."""
        T, K = x.shape
        N = weight.shape[1] if b_mn else weight.shape[0]
        W = self.world
        rows = T // W
        assert T % W == 0 and rows % 256 == 0 and rows <= self.max_rows and N <= self.max_cols
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
        scratch = self.rs_scratch[: rows * N].view(rows, N)
        self.rs_epoch += 1
        rc = _lib.lib().pb_gemm_tp_fused(
            _lib.c_int(2), _lib.ptr(x), _lib.ptr(weight), _lib.ptr(scratch), _lib.c_int(N), _lib.c_int(K),
            _lib.c_ll(x.stride(0)), _lib.c_ll(weight.stride(0)), _lib.c_ll(N), _lib.c_int(int(b_mn)),
            _lib.c_int(self.rank), _lib.c_int(W), _lib.c_int(rows), _lib.c_int(self.rs_epoch), None, None,
            self.rs_staging.pointer_array(), _lib.ptr(out), _lib.ptr(residual), self._flag_array(self.rs_flags),
            _lib.ptr(self.tile_flags), _lib.ptr(self.counters), _lib.c_int(0),
            _lib.ptr(_lib.err_word(x.device)), _lib.stream_ptr(),
        )
        _lib.check(rc, "pb_gemm_tp_fused(GEMM -> reduce-scatter)")
        return out

    def all_gather_rows(self, x_shard: torch.Tensor, ctas: int = 32) -> torch.Tensor:
        """Concatenation of every rank's ``[rows, cols]`` shard, by this package's peer-memory all-gather kernel
        (``csrc/peer.cu``: plain vector loads over NVLink, flag handshakes); the shard travels through the same
        peer-mapped buffer the fused all-gather -> GEMM publishes its input in."""
        rows, cols = x_shard.shape
        nbytes = rows * cols * x_shard.element_size()
        if x_shard.dtype != torch.bfloat16 or nbytes % 16 != 0 or rows > self.max_rows or cols > self.max_cols:
            out = torch.empty(self.world * rows, cols, dtype=x_shard.dtype, device=x_shard.device)
            dist.all_gather_into_tensor(out, x_shard.contiguous(), group=self.group)
            return out
        src = self.ag_src.tensor(torch.bfloat16, rows * cols).view(rows, cols)
        src.copy_(x_shard)
        out = torch.empty(self.world * rows, cols, dtype=torch.bfloat16, device=x_shard.device)
        self.gather_epoch += 1
        rc = _lib.lib().pb_peer_allgather(
            _lib.ptr(out), self.ag_src.pointer_array(), self._flag_array(self.gather_flags),
            _lib.ptr(self.gather_counter), _lib.ptr(_lib.err_word(x_shard.device)), _lib.c_ll(nbytes),
            _lib.c_int(self.rank), _lib.c_int(self.world), _lib.c_int(self.gather_epoch), _lib.c_int(ctas),
            _lib.stream_ptr())
        _lib.check(rc, "pb_peer_allgather")
        return out


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, tp: TPContext):
        y, _ = tp.ag_gemm(x_shard, weight)
        ctx.save_for_backward(x_shard)
        ctx.weight = weight  # parameters ride on ctx: saved-tensor hooks (checkpointing) would hand back a stand-in
        ctx.tp = tp
        weight._pb_direct_grad = True
        return y

    @staticmethod
    def backward(ctx, dy):
        (x_shard,) = ctx.saved_tensors
        weight = ctx.weight
        tp = ctx.tp
        dy = dy.contiguous()
        dx_shard = tp.gemm_rs(dy, weight, b_mn=True)  # [T, N_local] . [N_local, K] -> rows scattered
        x_full = tp.all_gather_rows(x_shard)
        mg = getattr(weight, "main_grad", None)
        if mg is not None and mg.dtype == torch.float32:
            gemm(dy, x_full, a_mn=True, b_mn=True, out=mg.view(weight.shape), accumulate=True)
        else:
            _accumulate_param_grad(weight, gemm(dy, x_full, a_mn=True, b_mn=True))
        return dx_shard, None, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual_shard, tp: TPContext):
        out = tp.gemm_rs(x, weight, residual=residual_shard)
        ctx.save_for_backward(x)
        ctx.weight = weight
        ctx.tp = tp
        ctx.has_res = residual_shard is not None
        weight._pb_direct_grad = True
        return out

    @staticmethod
    def backward(ctx, dout_shard):
        (x,) = ctx.saved_tensors
        weight = ctx.weight
        tp = ctx.tp
        dout_shard = dout_shard.contiguous()
        dx, gathered = tp.ag_gemm(dout_shard, weight, b_mn=True)  # gather(dOut) . W -> [T, K_local]
        rows = dout_shard.shape[0]
        gathered[tp.rank * rows : (tp.rank + 1) * rows].copy_(dout_shard)  # own rows are not copied by the kernel
        mg = getattr(weight, "main_grad", None)
        if mg is not None and mg.dtype == torch.float32:
            gemm(gathered, x, a_mn=True, b_mn=True, out=mg.view(weight.shape), accumulate=True)
        else:
            _accumulate_param_grad(weight, gemm(gathered, x, a_mn=True, b_mn=True))
        return dx, None, (dout_shard if ctx.has_res else None), None


class ColumnParallelLinear(nn.Module):
    """``weight`` holds this rank's ``out_features / tp`` rows. Input: token shard ``[T/tp, in]``; output
    ``[T, out/tp]``."""

    def __init__(self, in_features: int, out_features: int, tp: Optional[TPContext], tp_size: int = 1,
                 init_std: float = 0.02, device=None, dtype=None):
        super().__init__()
        assert out_features % tp_size == 0
        self.tp = tp
        self.weight = nn.Parameter(torch.empty(out_features // tp_size, in_features, device=device, dtype=dtype))
        nn.init.normal_(self.weight, std=init_std)

    def forward(self, x_shard):
        if self.tp is not None and x_shard.is_cuda and x_shard.dtype == torch.bfloat16:
            return _ColumnParallelFn.apply(x_shard, self.weight, self.tp)
        from .tp_reference import column_parallel_reference

        return column_parallel_reference(x_shard, self.weight, self.tp.group if self.tp is not None else None)


class RowParallelLinear(nn.Module):
    """``weight`` holds this rank's ``in_features / tp`` columns. Input ``[T, in/tp]``; output: token shard
    ``[T/tp, out]`` (+ residual shard)."""

    def __init__(self, in_features: int, out_features: int, tp: Optional[TPContext], tp_size: int = 1,
                 init_std: float = 0.02, device=None, dtype=None):
        super().__init__()
        assert in_features % tp_size == 0
        self.tp = tp
        self.weight = nn.Parameter(torch.empty(out_features, in_features // tp_size, device=device, dtype=dtype))
        nn.init.normal_(self.weight, std=init_std)

    def forward(self, x, residual_shard=None):
        if self.tp is not None and x.is_cuda and x.dtype == torch.bfloat16:
            return _RowParallelFn.apply(x, self.weight, residual_shard, self.tp)
        from .tp_reference import row_parallel_reference

        return row_parallel_reference(x, self.weight, residual_shard, self.tp.group if self.tp is not None else None)
