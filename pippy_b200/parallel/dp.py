"""Data-parallel gradient reduction for pipeline stages.

``GradReducer`` owns, per rank, a bf16 wire buffer in peer-mapped memory that mirrors the stage's flat fp32 gradient
buffer.  When the schedule reaches a stage's REDUCE_GRAD action (right after that stage's last backward or
weight-gradient pass) the stage's slice of the flat buffer is all-reduced across the data-parallel group by ONE
kernel that also applies the cast and the 1/replicas scale and moves the data with P2P loads and stores over NVLink
(``csrc/dp_allreduce.cu``).  The launch goes to a side stream, so the reduction of one stage runs under the backward of
the stages scheduled after it.  The reference leaves this to a wrapped DDP module whose reducer it pokes by hand
(pippy/_PipelineStage.py:409-450).

On CPU (tests) or for non-bf16/fp32 layouts the same interface falls back to ``dist.all_reduce``.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..optim import FlatParams
from ..utils import streamcheck


class GradReducer:
    def __init__(self, flat: FlatParams, dp_group: Optional[dist.ProcessGroup], max_ctas: int = 296,
                 average: bool = True):
        """``max_ctas`` bounds the kernel's grid (two thread blocks per SM by default: the three passes are
        bandwidth-bound and need the parallelism; the blocks need not be resident together, so a grid larger than
        what fits beside a running GEMM only waits its turn)."""
        self.flat = flat
        self.group = dp_group
        self.world = dist.get_world_size(dp_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(dp_group) if dist.is_initialized() else 0
        self.scale = (1.0 / self.world) if average else 1.0
        self.max_ctas = max_ctas
        self.epoch = 0
        self._ranges: Dict[int, Tuple[int, int]] = {}
        self.fused = (
            flat.grad.is_cuda and flat.grad.dtype == torch.float32 and self.world > 1 and self.world <= 8
        )
        self._stream = None
        self._pending = []
        if self.fused:
            from ..comm.symm import SymmetricBuffer

            n = (flat.numel + 7) // 8 * 8
            self.n_padded = n
            self.staging = SymmetricBuffer(n * 2, dp_group, flat.grad.device)
            self.flags = SymmetricBuffer(4096, dp_group, flat.grad.device)
            self.counter = torch.zeros(2, dtype=torch.int32, device=flat.grad.device)
            self._stream = torch.cuda.Stream(device=flat.grad.device)

    def _stage_range(self, stage) -> Tuple[int, int]:
        key = id(stage)
        r = self._ranges.get(key)
        if r is None:
            ids = {id(p) for p in stage.submod.parameters()}
            offs = [(o, p.numel()) for p, o in zip(self.flat.params, self.flat.offsets) if id(p) in ids]
            if not offs:
                r = (0, 0)
            else:
                lo = min(o for o, _ in offs)
                hi = max(o + n for o, n in offs)
                lo = lo // 8 * 8
                hi = min((hi + 7) // 8 * 8, self.flat.numel // 8 * 8 if self.flat.numel % 8 == 0 else hi)
                r = (lo, hi)
            self._ranges[key] = r
        return r

    def reduce_stage(self, stage) -> None:
        lo, hi = self._stage_range(stage)
        if hi <= lo or self.world == 1:
            return
        self.flat.fold_autograd_grads()
        self._reduce_range(lo, hi)

    def reduce_all(self) -> None:
        if self.world == 1:
            return
        self.flat.fold_autograd_grads()
        self._reduce_range(0, self.flat.numel)

    def _reduce_range(self, lo: int, hi: int) -> None:
        grad = self.flat.grad
        n = hi - lo
        if not self.fused or n % 8 != 0 or lo % 8 != 0:
            seg = grad[lo:hi]
            seg.mul_(self.scale)
            dist.all_reduce(seg, group=self.group)
            return
        cur = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(cur)
        self._stream.wait_event(ready)
        chk = streamcheck.tracker()
        if chk is not None:  # debug mode: the gradients were produced on `cur`, the reduction rewrites them on the side stream
            chk.write(f"grad@{id(self.flat)}", cur.cuda_stream)
            chk.ordered(cur.cuda_stream, self._stream.cuda_stream)
            chk.write(f"grad@{id(self.flat)}", self._stream.cuda_stream)
        with torch.cuda.stream(self._stream):
            self.epoch += 1
            grid = ctypes.c_int(0)
            stag = self.staging.pointer_array(lo * 2)
            flg = (ctypes.POINTER(ctypes.c_int) * self.world)()
            for i, ptr in enumerate(self.flags.ptrs):
                flg[i] = ctypes.cast(ctypes.c_void_p(ptr), ctypes.POINTER(ctypes.c_int))
            rc = _lib.lib().pb_dp_allreduce(
                ctypes.c_void_p(grad.data_ptr() + lo * 4), stag, flg, _lib.ptr(self.counter),
                _lib.ptr(_lib.err_word(grad.device)), _lib.c_ll(n), _lib.c_float(self.scale), _lib.c_int(self.rank),
                _lib.c_int(self.world), _lib.c_int(self.epoch),
                _lib.c_int(self.max_ctas), ctypes.byref(grid), ctypes.c_void_p(self._stream.cuda_stream),
            )
            _lib.check(rc, "pb_dp_allreduce")
            done = torch.cuda.Event()
            done.record(self._stream)
            self._pending.append(done)

    def finish(self) -> None:
        """Makes the current stream wait for every reduction launched so far."""
        cur = torch.cuda.current_stream() if self._stream is not None else None
        for ev in self._pending:
            cur.wait_event(ev)
        chk = streamcheck.tracker()
        if chk is not None and self._stream is not None and self._pending:
            chk.ordered(self._stream.cuda_stream, cur.cuda_stream)
        self._pending.clear()

    def check_read(self) -> None:
        """Debug mode only: declares that the current stream is about to read (or rescale) the gradients; raises
        ``StreamOrderError`` if a reduction is still in flight on the side stream (``finish()`` was not called)."""
        chk = streamcheck.tracker()
        if chk is not None and self._stream is not None:
            chk.read(f"grad@{id(self.flat)}", torch.cuda.current_stream().cuda_stream)
