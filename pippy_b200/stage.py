"""Per-rank stage runtime: receive buffers, point-to-point ops, per-microbatch forward and backward.

Reference: pippy/_PipelineStage.py (PipelineStageBase :72-176, p2p ops :178-341, compute :452-550, data-parallel
hooks :409-450, graph-derived topology :553-815).  Differences by design:

* every method takes the microbatch index explicitly, so any action order (1F1B, interleaved, zero-bubble)
  can drive a stage; the implicit counters of the reference remain as a convenience for in-order use;
* stage topology is a small table (which stage/output feeds each input, where each output goes), so skip
  connections work in both directions: gradients of an output consumed by several stages are summed;
* two stages on the same rank hand tensors over directly instead of sending to self;
* the backward can be split into an input-gradient and a weight-gradient half.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn

from ._debug import map_debug_info
from .backward import (
    _null_coalesce_accumulate,
    stage_backward,
    stage_backward_input,
    stage_backward_weight,
)
from .utils.tree import flatten_args

logger = logging.getLogger("pippy_b200")


class RootArgPlaceholder:
    """Marks a stage input that is a model input supplied by the caller of ``step()``."""

    def __repr__(self) -> str:
        return "RootArgPlaceholder()"


@dataclass
class RecvInfo:
    """One tensor a stage receives: which stage produces it and the buffer it lands in."""

    input_name: str
    source: int
    buffer: torch.Tensor

    def __repr__(self) -> str:
        return f"RecvInfo(input={self.input_name}, source={self.source}, shape={tuple(self.buffer.shape)})"


@dataclass
class TensorMeta:
    shape: torch.Size
    dtype: torch.dtype

    @staticmethod
    def of(t: torch.Tensor) -> "TensorMeta":
        return TensorMeta(t.shape, t.dtype)


@dataclass
class InputSpec:
    """Where input ``i`` of a stage comes from: ``source`` stage and its output index; None = model input."""

    name: str
    source: Optional[int]
    source_output: int
    meta: Optional[TensorMeta]


class PipelineStageBase:
    """State and mechanics shared by traced and manual stages."""

    def __init__(
        self,
        submodule: nn.Module,
        stage_index: int,
        num_stages: int,
        device: torch.device,
        group: Optional[dist.ProcessGroup] = None,
    ):
        if stage_index >= num_stages:
            raise ValueError(f"Stage index {stage_index} is out of range of {num_stages} stages")
        self.submod = submodule
        self.stage_index = stage_index
        self.num_stages = num_stages
        self.device = torch.device(device)
        self.group = group
        if dist.is_available() and dist.is_initialized():
            self.group_rank = dist.get_rank(group)
            self.group_size = dist.get_world_size(group)
        else:  # single-process use (tests, local execution)
            self.group_rank = 0
            self.group_size = 1
        if self.group_size > num_stages:
            raise RuntimeError(
                f"Pipeline group size {self.group_size} cannot be larger than number of stages {num_stages}"
            )
        # stage i lives on group rank i % group_size (interleaving wraps around)
        self.stage_index_to_group_rank: Dict[int, int] = {i: i % self.group_size for i in range(num_stages)}

        # topology, filled by subclasses
        self.input_specs: List[InputSpec] = []
        self.output_metas: List[TensorMeta] = []
        self.output_dests: Dict[int, List[int]] = {}  # output idx -> consumer stages
        self.chunks: Optional[int] = None
        self.has_backward = False
        self.keep_outputs = True  # the schedule clears this when its caller does not want the merged output
        self.scale_grads_by: Optional[float] = None

        # run-time state
        self.fwd_cache: Dict[int, Tuple[Tuple[Any, ...], List[Any]]] = {}
        self.output_chunks: Dict[int, Any] = {}
        self.args_recv_info: Dict[int, Tuple[Union[RecvInfo, RootArgPlaceholder], ...]] = {}
        self.grad_recv_info: Dict[int, Dict[Tuple[int, int], RecvInfo]] = {}
        self.grads_input: Dict[int, List[Optional[torch.Tensor]]] = {}
        self.local_inputs: Dict[int, Dict[int, torch.Tensor]] = {}       # mb -> input idx -> tensor handed over
        self.local_out_grads: Dict[int, Dict[Tuple[int, int], torch.Tensor]] = {}  # mb -> (out idx, consumer)
        self.dw_plans: Dict[int, Any] = {}
        self.fwd_chunk_id = 0
        self.bwd_chunk_id = 0
        self._dp_wrapper_configured_last = True
        self.link_groups = None  # comm.p2p.LinkGroups, installed by the schedule

    # ------------------------------------------------------------------ properties
    @property
    def is_first(self) -> bool:
        return self.stage_index == 0

    @property
    def is_last(self) -> bool:
        return self.stage_index == self.num_stages - 1

    def rank_of_stage(self, stage: int) -> int:
        return self.stage_index_to_group_rank[stage]

    def set_placement(self, stage_to_rank: Dict[int, int]) -> None:
        """Replaces the wrap-around stage -> group-rank map (stage i on rank i % group_size, reference
        _PipelineStage.py:129-136) by another one, e.g. the V shape of ``schedules.generators.v_placement``.  Must
        be the same on every rank and is set before a schedule is built on the stage."""
        if sorted(stage_to_rank) != list(range(self.num_stages)):
            raise ValueError(f"placement must map stages 0..{self.num_stages - 1}")
        if any(not 0 <= r < self.group_size for r in stage_to_rank.values()):
            raise ValueError(f"placement names a rank outside the pipeline group of {self.group_size}")
        if stage_to_rank[self.stage_index] != self.group_rank:
            raise ValueError(
                f"placement puts stage {self.stage_index} on rank {stage_to_rank[self.stage_index]}, but it was "
                f"built on rank {self.group_rank}"
            )
        self.stage_index_to_group_rank = dict(stage_to_rank)
        # which inputs arrive over the wire depends on the placement: receive buffers are rebuilt on next use
        chunks, self.chunks = self.chunks, None
        self.args_recv_info = {}
        self.grad_recv_info = {}
        if chunks is not None:
            self._prepare_forward_infra(chunks)

    def _global_rank(self, group_rank: int) -> int:
        if self.group is None:
            return group_rank
        return dist.get_global_rank(self.group, group_rank)

    def is_local_stage(self, stage: int) -> bool:
        return self.rank_of_stage(stage) == self.group_rank

    def _link_group(self, producer_rank: int, consumer_rank: int, kind: str):
        """Process group of the directed link producer -> consumer for forward ("F") transfers, or of the reverse
        direction for gradient ("B") transfers; the pipeline group when no per-link groups were installed."""
        if self.link_groups is not None:
            if kind == "F":
                g = self.link_groups.get(producer_rank, consumer_rank, "F")
            else:
                g = self.link_groups.get(consumer_rank, producer_rank, "B")
            if g is not None:
                return g
        return self.group

    # ------------------------------------------------------------------ buffers
    def _prepare_forward_infra(self, num_microbatches: int) -> None:
        """Allocates one receive buffer per (microbatch, remote input)."""
        if self.chunks == num_microbatches and self.args_recv_info:
            return
        self.chunks = num_microbatches
        self.args_recv_info = {}
        self.grad_recv_info = {}
        for mb in range(num_microbatches):
            infos: List[Union[RecvInfo, RootArgPlaceholder]] = []
            for spec in self.input_specs:
                if spec.source is None:
                    infos.append(RootArgPlaceholder())
                elif self.is_local_stage(spec.source):
                    infos.append(RootArgPlaceholder())  # filled by a local hand-over, never received
                else:
                    assert spec.meta is not None
                    buf = torch.empty(spec.meta.shape, dtype=spec.meta.dtype, device=self.device)
                    infos.append(RecvInfo(spec.name, spec.source, buf))
            self.args_recv_info[mb] = tuple(infos)

    def _grad_recv_infos(self, mb: int) -> Dict[Tuple[int, int], RecvInfo]:
        infos = self.grad_recv_info.get(mb)
        if infos is None:
            infos = {}
            for out_idx, consumers in self.output_dests.items():
                meta = self.output_metas[out_idx]
                if not meta.dtype.is_floating_point:
                    continue
                for dst in consumers:
                    if self.is_local_stage(dst):
                        continue
                    buf = torch.empty(meta.shape, dtype=meta.dtype, device=self.device)
                    infos[(out_idx, dst)] = RecvInfo(f"grad_out{out_idx}_from{dst}", dst, buf)
            self.grad_recv_info[mb] = infos
        return infos

    # ------------------------------------------------------------------ p2p ops
    def get_fwd_recv_ops(self, mb: Optional[int] = None, source: Optional[int] = None) -> List[dist.P2POp]:
        """irecv ops for the remote inputs of microbatch ``mb`` (optionally only those produced by ``source``)."""
        mb = self.fwd_chunk_id if mb is None else mb
        ops: List[dist.P2POp] = []
        for info in self.args_recv_info[mb]:
            if not isinstance(info, RecvInfo) or (source is not None and info.source != source):
                continue
            src_rank = self.rank_of_stage(info.source)
            peer = self._global_rank(src_rank)
            ops.append(dist.P2POp(dist.irecv, info.buffer, peer, self._link_group(src_rank, self.group_rank, "F")))
        return ops

    def get_bwd_recv_ops(self, mb: Optional[int] = None, source: Optional[int] = None) -> List[dist.P2POp]:
        if not self.has_backward or self.is_last:
            return []
        mb = self.bwd_chunk_id if mb is None else mb
        ops: List[dist.P2POp] = []
        for (_, dst), info in sorted(self._grad_recv_infos(mb).items()):
            if source is not None and dst != source:
                continue
            dst_rank = self.rank_of_stage(dst)
            peer = self._global_rank(dst_rank)
            ops.append(dist.P2POp(dist.irecv, info.buffer, peer, self._link_group(self.group_rank, dst_rank, "B")))
        return ops

    def get_fwd_send_ops(self, mb: Optional[int] = None) -> List[dist.P2POp]:
        """isend ops for every (output, remote consumer stage) of microbatch ``mb``, consumers ascending."""
        mb = (self.fwd_chunk_id - 1) if mb is None else mb
        outputs = getattr(self, "_sent_outputs", {}).get(mb)
        if outputs is None:
            return []
        ops: List[Tuple[int, int, dist.P2POp]] = []
        for out_idx, consumers in self.output_dests.items():
            out = outputs[out_idx]
            for dst in consumers:
                if self.is_local_stage(dst):
                    continue
                dst_rank = self.rank_of_stage(dst)
                peer = self._global_rank(dst_rank)
                ops.append((dst, out_idx, dist.P2POp(dist.isend, out.detach().contiguous(), peer,
                                                     self._link_group(self.group_rank, dst_rank, "F"))))
        ops.sort(key=lambda t: (t[0], t[1]))
        return [op for _, _, op in ops]

    def get_bwd_send_ops(self, mb: Optional[int] = None) -> List[dist.P2POp]:
        if not self.has_backward or self.is_first:
            return []
        mb = (self.bwd_chunk_id - 1) if mb is None else mb
        grads = self.grads_input[mb]
        ops: List[Tuple[int, int, dist.P2POp]] = []
        for idx, (spec, grad) in enumerate(zip(self.input_specs, grads)):
            if spec.source is None or self.is_local_stage(spec.source):
                continue
            is_float = spec.meta is not None and spec.meta.dtype.is_floating_point
            if grad is None and is_float:
                # A floating-point input that nothing differentiable depends on (an attention mask turned into
                # additive form on an earlier stage, a dropped branch): the producer has posted a receive for its
                # gradient all the same, since the two sides cannot know this before running, so zeros are sent.
                # The reference refuses such a boundary (pippy/_PipelineStage.py:336-340).
                if not hasattr(self, "_zero_grads"):
                    self._zero_grads: Dict[int, torch.Tensor] = {}
                grad = self._zero_grads.get(idx)
                if grad is None:
                    grad = torch.zeros(spec.meta.shape, dtype=spec.meta.dtype, device=self.device)
                    self._zero_grads[idx] = grad
            if grad is None:
                continue
            src_rank = self.rank_of_stage(spec.source)
            peer = self._global_rank(src_rank)
            ops.append((spec.source, idx, dist.P2POp(dist.isend, grad.contiguous(), peer,
                                                     self._link_group(src_rank, self.group_rank, "B"))))
        for idx, grad in enumerate(grads):
            if grad is not None and idx < len(self.input_specs) and self.input_specs[idx].source is None:
                pass  # gradient of a model input: nothing to send
        ops.sort(key=lambda t: (t[0], t[1]))
        return [op for _, _, op in ops]

    # ------------------------------------------------------------------ local hand-over (same-rank stages)
    def local_forward_targets(self) -> List[Tuple[int, int]]:
        """(output idx, consumer stage) pairs whose consumer lives on this rank."""
        return [(o, d) for o, ds in self.output_dests.items() for d in ds if self.is_local_stage(d)]

    def set_local_input(self, mb: int, source_stage: int, source_output: int, value: torch.Tensor) -> None:
        for idx, spec in enumerate(self.input_specs):
            if spec.source == source_stage and spec.source_output == source_output:
                t = value.detach()
                if self.has_backward and t.is_floating_point():
                    t = t.requires_grad_(True)
                self.local_inputs.setdefault(mb, {})[idx] = t

    def set_local_out_grad(self, mb: int, out_idx: int, consumer: int, grad: Optional[torch.Tensor]) -> None:
        if grad is not None:
            self.local_out_grads.setdefault(mb, {})[(out_idx, consumer)] = grad

    # ------------------------------------------------------------------ compute
    def _compose_inputs(self, mb: int, args: Tuple[Any, ...]) -> List[Any]:
        infos = self.args_recv_info[mb]
        root = iter(args)
        composite: List[Any] = []
        local = self.local_inputs.get(mb, {})
        for idx, (spec, info) in enumerate(zip(self.input_specs, infos)):
            if isinstance(info, RecvInfo):
                buf = info.buffer
                if self.has_backward and buf.is_floating_point() and not buf.requires_grad:
                    buf.requires_grad_(True)
                composite.append(buf)
            elif spec.source is not None:
                if idx not in local:
                    raise RuntimeError(
                        f"[{self.stage_index}] microbatch {mb}: input {spec.name!r} from local stage {spec.source} "
                        "was not handed over before forward"
                    )
                composite.append(local[idx])
            else:
                try:
                    composite.append(next(root))
                except StopIteration:
                    raise RuntimeError(
                        f"[{self.stage_index}] microbatch {mb}: not enough positional model inputs; the stage expects "
                        f"{sum(1 for s in self.input_specs if s.source is None)}"
                    ) from None
        composite.extend(root)  # extra positional args pass through (first stage called with more args)
        return composite

    def _compose_inputs_for_forward(self, mb: int, args: Tuple[Any, ...]) -> List[Any]:
        return self._compose_inputs(mb, args)

    def forward_maybe_with_nosync(self, *args, **kwargs):
        from torch.nn.parallel import DistributedDataParallel

        if isinstance(self.submod, DistributedDataParallel):
            with self.submod.no_sync():
                return self.submod(*args, **kwargs)
        return self.submod(*args, **kwargs)

    def forward_one_chunk(self, *call_args, **call_kwargs):
        """``forward_one_chunk(mb, args, kwargs)`` or, in order, ``forward_one_chunk(args, kwargs)``."""
        mb, args, kwargs = self._parse_chunk_call(call_args, call_kwargs, forward=True)
        if self.chunks is None or mb not in self.args_recv_info:
            raise RuntimeError(
                f"[{self.stage_index}] microbatch {mb} has no receive info; did the schedule prepare "
                f"{self.chunks} microbatches?"
            )
        composite_args = self._compose_inputs_for_forward(mb, tuple(args))
        try:
            output = self.forward_maybe_with_nosync(*composite_args, **kwargs)
        except Exception as e:
            raise RuntimeError(
                f"""
            [{self.stage_index}] failed to run forward:
            args: {map_debug_info(composite_args)}
            kwargs: {map_debug_info(kwargs)}
            """
            ) from e
        if isinstance(output, list):
            output = tuple(output)
        output_tuple = output if isinstance(output, tuple) else (output,)
        # what outlives the backward must not pin the autograd graph: keep detached views only
        def _detached(o):
            return o.detach() if isinstance(o, torch.Tensor) else o

        if self.is_last and self.keep_outputs:
            self.output_chunks[mb] = (
                tuple(_detached(o) for o in output) if isinstance(output, tuple) else _detached(output)
            )
        flat_inputs = flatten_args(composite_args) + flatten_args(kwargs)
        self.fwd_cache[mb] = (output_tuple, flat_inputs)
        if not hasattr(self, "_sent_outputs"):
            self._sent_outputs: Dict[int, Tuple[Any, ...]] = {}
        if any(self.output_dests.values()):  # the last stage sends nothing: do not pin its outputs
            self._sent_outputs[mb] = tuple(_detached(o) for o in output_tuple)
        self.fwd_chunk_id = mb + 1
        if logger.isEnabledFor(logging.DEBUG):  # the rendering itself costs more than a small stage's launches
            logger.debug("[%d] Forwarded chunk %d, outputs: %s", self.stage_index, mb, map_debug_info(output))
        return output

    def _parse_chunk_call(self, call_args, call_kwargs, forward: bool):
        if call_args and isinstance(call_args[0], int) and not isinstance(call_args[0], bool):
            mb = call_args[0]
            rest = call_args[1:]
        else:
            mb = self.fwd_chunk_id if forward else self.bwd_chunk_id
            rest = call_args
        args = rest[0] if len(rest) > 0 and rest[0] is not None else call_kwargs.pop("args", ())
        kwargs = rest[1] if len(rest) > 1 and rest[1] is not None else call_kwargs.pop("kwargs", None)
        return mb, (args or ()), (kwargs or {})

    def _collect_output_grads(self, mb: int, outputs: Tuple[Any, ...]) -> Tuple[Optional[torch.Tensor], ...]:
        remote = self._grad_recv_infos(mb)
        local = self.local_out_grads.pop(mb, {})
        grads: List[Optional[torch.Tensor]] = []
        for out_idx in range(len(outputs)):
            acc: Optional[torch.Tensor] = None
            for dst in self.output_dests.get(out_idx, []):
                g = local.get((out_idx, dst))
                if g is None:
                    info = remote.get((out_idx, dst))
                    g = info.buffer if info is not None else None
                acc = _null_coalesce_accumulate(acc, g)
            grads.append(acc)
        return tuple(grads)

    def backward_one_chunk(self, mb: Optional[int] = None, loss=None, full_backward: bool = True) -> None:
        """Backward of microbatch ``mb``. With ``full_backward=False`` only input gradients are produced now and
        :meth:`backward_weight_one_chunk` must follow."""
        mb = self.bwd_chunk_id if mb is None else mb
        self._check_chunk_id(mb)
        outputs, inputs = self.fwd_cache.pop(mb)
        if self.is_last:
            if loss is None:
                raise RuntimeError(f"[{self.stage_index}] the last stage needs the loss of microbatch {mb} to run backward")
            bwd_outputs: Any = (loss,)
            out_grads: Any = None
        else:
            bwd_outputs = outputs
            out_grads = self._collect_output_grads(mb, outputs)
        if full_backward:
            target = loss if self.is_last else bwd_outputs
            grads_input = self._run_backward_with_dp(lambda: stage_backward(target, out_grads, inputs), target)
        else:
            flat_out = list(bwd_outputs)
            flat_grads = None if out_grads is None else list(out_grads)
            grads_input, plan = stage_backward_input(flat_out, flat_grads, inputs, self.submod.parameters())
            self.dw_plans[mb] = plan
        n_in = len(self.input_specs)
        self.grads_input[mb] = list(grads_input[:n_in]) + [None] * max(0, n_in - len(grads_input))
        # gradients were read; release them so recv buffers do not accumulate across microbatches
        for v in inputs:
            if isinstance(v, torch.Tensor) and v.grad is not None and v.is_leaf and not isinstance(v, nn.Parameter):
                v.grad = None
        self.bwd_chunk_id = mb + 1
        logger.debug("[%d] Backwarded chunk %d", self.stage_index, mb)

    def backward_weight_one_chunk(self, mb: int) -> None:
        plan = self.dw_plans.pop(mb, None)
        if plan is None:
            raise RuntimeError(f"[{self.stage_index}] no deferred weight gradients for microbatch {mb}")
        stage_backward_weight(self.submod.parameters(), plan)

    def _check_chunk_id(self, mb: int) -> None:
        if mb not in self.fwd_cache:
            raise RuntimeError(
                f"[{self.stage_index}] backward of microbatch {mb} requested but its forward is not cached "
                f"(cached: {sorted(self.fwd_cache)})"
            )

    def clear_runtime_states(self) -> None:
        """Resets per-step state; receive buffers keep their storage but drop accumulated gradients."""
        self.fwd_cache.clear()
        self.output_chunks.clear()
        self.grads_input.clear()
        self.local_inputs.clear()
        self.local_out_grads.clear()
        self.dw_plans.clear()
        if hasattr(self, "_sent_outputs"):
            self._sent_outputs.clear()
        self.fwd_chunk_id = 0
        self.bwd_chunk_id = 0
        for infos in self.args_recv_info.values():
            for info in infos:
                if isinstance(info, RecvInfo):
                    info.buffer.grad = None

    # ------------------------------------------------------------------ data-parallel wrappers
    def _configure_data_parallel_mode(self, last_backward: bool) -> None:
        """Tells a DDP/FSDP-wrapped submodule whether the coming backward is the one that must reduce
        gradients (reference _PipelineStage.py:409-450)."""
        self._dp_wrapper_configured_last = last_backward
        try:
            from torch.distributed.fsdp import FSDPModule
        except Exception:  # pragma: no cover - older torch
            FSDPModule = ()
        if FSDPModule and isinstance(self.submod, FSDPModule):
            self.submod.set_is_last_backward(last_backward)
            self.submod.set_requires_gradient_sync(last_backward)

    def _run_backward_with_dp(self, fn, outputs_for_ddp):
        from torch.nn.parallel import DistributedDataParallel

        if isinstance(self.submod, DistributedDataParallel):
            if self._dp_wrapper_configured_last:
                # stage_backward bypasses DDP.forward, so arm the reducer by hand for this backward
                from torch.nn.parallel.distributed import _find_tensors

                self.submod.reducer.prepare_for_backward(list(_find_tensors(outputs_for_ddp)))
                return fn()
            with self.submod.no_sync():
                return fn()
        return fn()

    def scale_grads(self, divisor: float) -> None:
        """Divides every parameter gradient by ``divisor`` (used when losses are means over microbatches)."""
        if divisor == 1:
            return
        for p in self.submod.parameters():
            if p.grad is not None:
                p.grad.div_(divisor)
            mg = getattr(p, "main_grad", None)
            if mg is not None:
                mg.div_(divisor)

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}(stage={self.stage_index}/{self.num_stages}, rank={self.group_rank})"
