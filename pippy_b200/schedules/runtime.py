"""Executes a schedule (a per-rank action list) on this rank's stages, and the public schedule classes.

Public surface follows the reference (pippy/PipelineSchedule.py): ``ScheduleGPipe`` / ``Schedule1F1B`` take one
stage, ``ScheduleLoopedBFS`` / ``ScheduleInterleaved1F1B`` a list of local stages, all expose
``step(*args, target=None, losses=None, **kwargs)``.  ``ScheduleInterleavedZeroBubble`` adds the split-backward
schedule the reference lacks (upstream torch/distributed/pipelining/schedules.py:2621-2810).

How it differs from the reference's imperative loops:
* one interpreter for every schedule; schedules are data (``actions.py``) produced by pure functions;
* receives are posted ahead of the compute that needs them and only waited right before it, sends are never
  waited until the end of the step: on NCCL both run on the communicator's own stream, so activations and
  gradients move while the stage computes;
* stages that share a rank exchange tensors by reference;
* every compute action can be timed (CUDA events or host clock) to report the measured bubble.
"""
from __future__ import annotations

import logging
import time
from collections import defaultdict
from datetime import timedelta
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
from torch.profiler import record_function

from ..microbatch import TensorChunkSpec, merge_chunks, split_args_kwargs_into_chunks
from ..stage import PipelineStageBase
from . import generators
from .actions import Action, Op, Schedule, add_send_recv, format_schedule, validate

logger = logging.getLogger("pippy_b200")


class ScheduleTimeout(RuntimeError):
    """A communication wait exceeded the schedule's time limit; the message names the blocked action."""


def sorted_batch_isend_irecv(p2p_ops: List[dist.P2POp]) -> Dict[int, Any]:
    """Issues the ops grouped by peer, peers in ascending order, one batch per peer; returns ``{peer: work}``.
    A fixed issue order across ranks avoids deadlocks when a stage talks to several peers (skip connections)
    (reference PipelineSchedule.py:200-222)."""
    by_peer: Dict[Any, List[dist.P2POp]] = defaultdict(list)
    for op in p2p_ops:
        by_peer[(op.peer, id(op.group))].append(op)  # a batch must stay inside one process group
    works: Dict[Any, Any] = {}
    for key in sorted(by_peer, key=lambda k: k[0]):
        reqs = dist.batch_isend_irecv(by_peer[key])
        work = reqs[-1] if len(reqs) == 1 else _WorkGroup(reqs)
        works[key[0] if key[0] not in works else key] = work
    return works


class _WorkGroup:
    def __init__(self, works):
        self.works = list(works)

    def wait(self, timeout: Optional[timedelta] = None):
        for w in self.works:
            if timeout is None:
                w.wait()
            else:
                w.wait(timeout)


class _Timer:
    """Times compute actions with CUDA events on the current stream, or the host clock on CPU."""

    def __init__(self, cuda: bool):
        self.cuda = cuda
        self.records: List[Tuple[Action, Any, Any]] = []
        self.t_begin = None
        self.t_end = None

    def begin_step(self):
        self.records.clear()
        self.t_begin = self._now()

    def end_step(self):
        self.t_end = self._now()

    def _now(self):
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    def start(self):
        return self._now()

    def stop(self, action: Action, t0):
        self.records.append((action, t0, self._now()))

    def summary(self) -> Dict[str, Any]:
        if self.cuda:
            torch.cuda.synchronize()
            wall = self.t_begin.elapsed_time(self.t_end) * 1e-3
            durs = [(a, s.elapsed_time(e) * 1e-3) for a, s, e in self.records]
            starts = [self.t_begin.elapsed_time(s) * 1e-3 for _, s, _ in self.records]
        else:
            wall = self.t_end - self.t_begin
            durs = [(a, e - s) for a, s, e in self.records]
            starts = [s - self.t_begin for _, s, _ in self.records]
        busy = sum(d for _, d in durs)
        per_op: Dict[str, float] = defaultdict(float)
        per_stage: Dict[Tuple[int, str], List[float]] = defaultdict(list)
        for a, d in durs:
            per_op[a.op.value] += d
            per_stage[(a.stage, a.op.value)].append(d)
        return {
            # mean duration of one microbatch's F / B / I / W on each local stage: what a cost-aware schedule needs
            "per_stage_op_mean_s": {f"{s}:{o}": sum(v) / len(v) for (s, o), v in per_stage.items()},
            "wall_s": wall,
            "busy_s": busy,
            "bubble": (1.0 - busy / wall) if wall > 0 else 0.0,
            "per_op_s": dict(per_op),
            "actions": [(str(a), d) for a, d in durs],
            "timeline": [(str(a), t0, t0 + d) for (a, d), t0 in zip(durs, starts)],
        }


class PipelineSchedule:
    """Base of all schedules: input checking/splitting, loss bookkeeping, the action interpreter."""

    def __init__(
        self,
        stages: Sequence[PipelineStageBase],
        n_microbatches: int,
        loss_fn: Optional[Callable[..., torch.Tensor]] = None,
        output_merge_spec: Optional[Any] = None,
        args_chunk_spec: Optional[Tuple[Any, ...]] = None,
        kwargs_chunk_spec: Optional[Dict[str, Any]] = None,
        scale_grads: bool = False,
        grad_reducer: Optional[Any] = None,
        p2p_timeout_s: Optional[float] = None,
        record_timing: bool = False,
        use_link_groups: bool = True,
        return_outputs: bool = True,
    ):
        self._stages = sorted(stages, key=lambda s: s.stage_index)
        self._stage_by_index = {s.stage_index: s for s in self._stages}
        self._n_microbatches = n_microbatches
        self._loss_fn = loss_fn
        self._output_merge_spec = output_merge_spec
        self._has_backward = loss_fn is not None
        self._internal_losses: Dict[int, torch.Tensor] = {}
        self.scale_grads = scale_grads
        self.grad_reducer = grad_reducer
        self.p2p_timeout_s = p2p_timeout_s
        self.record_timing = record_timing
        # A training loop that only wants the losses passes False: the last stage then neither keeps every
        # microbatch's output alive until the end of the step nor concatenates them (for a language model that is
        # the full [batch, seq, vocab] logits, twice).
        self.return_outputs = return_outputs
        self.last_step_stats: Optional[Dict[str, Any]] = None
        first = self._stages[0]
        self.pp_group_size = first.group_size
        self.rank = first.group_rank
        self.num_stages = first.num_stages
        self._num_local = len(self._stages)
        pipe_info = getattr(first, "pipe_info", None)
        self._args_chunk_spec = args_chunk_spec if args_chunk_spec is not None else getattr(pipe_info, "args_chunk_spec", None)
        self._kwargs_chunk_spec = (
            kwargs_chunk_spec if kwargs_chunk_spec is not None else getattr(pipe_info, "kwargs_chunk_spec", None)
        )
        for st in self._stages:
            st.has_backward = self._has_backward
            st.keep_outputs = return_outputs
            st._prepare_forward_infra(n_microbatches)
        self.link_groups = None
        if dist.is_available() and dist.is_initialized() and self.pp_group_size > 1 and use_link_groups:
            from ..comm.p2p import LinkGroups, pipeline_links

            links = pipeline_links(self.num_stages, self.pp_group_size, self._topology(),
                                   first.stage_index_to_group_rank)
            # communicators are expensive: stages built once keep theirs across schedule objects
            self.link_groups = first.link_groups if first.link_groups is not None else LinkGroups(first.group, links)
            for st in self._stages:
                st.link_groups = self.link_groups
        self._actions: Optional[List[Action]] = None
        self.pipeline_order: Optional[Schedule] = None
        self.pipeline_order_with_comms: Optional[Schedule] = None

    # ------------------------------------------------------------------ schedule construction
    def _compute_order(self) -> Schedule:
        raise NotImplementedError

    def _stage_to_rank(self, stage: int) -> int:
        return self._stages[0].stage_index_to_group_rank[stage]

    def _topology(self) -> Optional[Dict[int, List[int]]]:
        topo = getattr(self._stages[0], "global_dests", None)
        return topo

    def _build(self) -> None:
        order = self._compute_order()
        validate(order, self.num_stages, self._n_microbatches, self._stage_to_rank)
        if self.grad_reducer is not None and self._has_backward:
            order = generators.with_reduce_grad(order)
        self.pipeline_order = order
        self.pipeline_order_with_comms = add_send_recv(order, self._stage_to_rank, self.num_stages, self._topology())
        self._actions = self.pipeline_order_with_comms[self.rank]
        last_bwd: Dict[int, int] = {}
        for a in self._actions:
            if a.op in (Op.B, Op.I):
                last_bwd[a.stage] = a.mb
        self._last_backward_mb = last_bwd
        logger.debug("schedule for rank %d:\n%s", self.rank, " ".join(str(a) for a in self._actions))

    def load_actions(self, schedule: Schedule) -> None:
        """Replaces the generated order with a user-provided one (for example read with ``actions.load_csv``).
        Communication actions are added if the schedule has none."""
        has_comm = any(a.op.is_comm for acts in schedule.values() for a in acts)
        self.pipeline_order = schedule
        self.pipeline_order_with_comms = (
            schedule if has_comm else add_send_recv(schedule, self._stage_to_rank, self.num_stages, self._topology())
        )
        self._actions = self.pipeline_order_with_comms[self.rank]
        self._last_backward_mb = {a.stage: a.mb for a in self._actions if a.op in (Op.B, Op.I)}

    def describe(self) -> str:
        if self._actions is None:
            self._build()
        return format_schedule(self.pipeline_order_with_comms)

    # ------------------------------------------------------------------ inputs / outputs / losses
    def _check_inputs(self, arg_mbs, kwarg_mbs, target_mbs, losses):
        def check_list(mbs, name):
            if not isinstance(mbs, list):
                raise TypeError(f"{name} must be a list but got a {type(mbs)}")
            if len(mbs) != self._n_microbatches:
                raise ValueError(f"Expecting {self._n_microbatches} {name} but got {len(mbs)}")

        if arg_mbs is not None:
            check_list(arg_mbs, "arg_mbs")
        else:
            arg_mbs = [()] * self._n_microbatches
        if kwarg_mbs is not None:
            check_list(kwarg_mbs, "kwarg_mbs")
        else:
            kwarg_mbs = [{}] * self._n_microbatches
        if target_mbs is not None:
            check_list(target_mbs, "target_mbs")
        if losses is not None and not isinstance(losses, list):
            raise TypeError(f"losses must be a list but got a {type(losses)}")
        return arg_mbs, kwarg_mbs

    def _split_inputs(self, args: Tuple[Any, ...], kwargs: Optional[Dict[str, Any]]):
        if args or kwargs:
            args_split, kwargs_split = split_args_kwargs_into_chunks(
                args, kwargs, self._n_microbatches, self._args_chunk_spec, self._kwargs_chunk_spec
            )
            return args_split, kwargs_split
        return [()] * self._n_microbatches, [{}] * self._n_microbatches

    def _merge_outputs(self, output_chunks: List[Any]) -> Any:
        return merge_chunks(output_chunks, self._output_merge_spec)

    def _maybe_compute_loss(self, stage: PipelineStageBase, output, target_mbs, mb: int) -> None:
        if stage.is_last and self._has_backward:
            if target_mbs is None:
                raise RuntimeError("a loss function was given, so the rank holding the last stage must pass `target`")
            loss = self._loss_fn(output, target_mbs[mb])
            self._internal_losses[mb] = loss
            logger.debug("[%d] loss of microbatch %d: %s", stage.stage_index, mb, loss)

    def _maybe_get_loss(self, stage: PipelineStageBase, mb: int):
        if stage.is_last and self._has_backward:
            if mb not in self._internal_losses:
                raise RuntimeError(
                    f"Loss of microbatch {mb} is not available; available: {sorted(self._internal_losses)}"
                )
            return self._internal_losses[mb]
        return None

    def _update_losses(self, losses: Optional[List[Any]]) -> None:
        holds_last = any(s.is_last for s in self._stages)
        if holds_last and losses is not None and self._has_backward:
            if len(self._internal_losses) != self._n_microbatches:
                raise RuntimeError(
                    f"Expecting {self._n_microbatches} losses but got {len(self._internal_losses)}"
                )
            losses.clear()
            losses.extend(self._internal_losses[mb] for mb in range(self._n_microbatches))
        self._internal_losses.clear()

    # ------------------------------------------------------------------ interpreter
    def _wait(self, works, action: Action) -> None:
        for w in works:
            if self.p2p_timeout_s is None:
                w.wait()
            else:
                try:
                    w.wait(timedelta(seconds=self.p2p_timeout_s))
                except Exception as e:  # gloo raises RuntimeError, NCCL DistBackendError
                    raise ScheduleTimeout(
                        f"rank {self.rank}: waiting for the transfers of {action} exceeded {self.p2p_timeout_s}s "
                        f"({type(e).__name__}: {e})"
                    ) from e

    def _step_microbatches(self, arg_mbs=None, kwarg_mbs=None, target_mbs=None, losses=None) -> None:
        arg_mbs, kwarg_mbs = self._check_inputs(arg_mbs, kwarg_mbs, target_mbs, losses)
        if self._actions is None:
            self._build()
        stages = self._stage_by_index
        pending_f: Dict[Tuple[int, int], List[Any]] = defaultdict(list)
        pending_b: Dict[Tuple[int, int], List[Any]] = defaultdict(list)
        send_works: List[Any] = []
        timer = None
        if self.record_timing:
            timer = _Timer(self._stages[0].device.type == "cuda")
            timer.begin_step()

        for action in self._actions:
            st = stages[action.stage]
            mb = action.mb
            op = action.op
            if op == Op.RECV_F:
                ops = st.get_fwd_recv_ops(mb, source=action.peer)
                if ops:
                    pending_f[(action.stage, mb)].extend(sorted_batch_isend_irecv(ops).values())
            elif op == Op.RECV_B:
                ops = st.get_bwd_recv_ops(mb, source=action.peer)
                if ops:
                    pending_b[(action.stage, mb)].extend(sorted_batch_isend_irecv(ops).values())
            elif op == Op.SEND_F:
                ops = st.get_fwd_send_ops(mb)
                if ops:
                    send_works.extend(sorted_batch_isend_irecv(ops).values())
            elif op == Op.SEND_B:
                ops = st.get_bwd_send_ops(mb)
                if ops:
                    send_works.extend(sorted_batch_isend_irecv(ops).values())
            elif op == Op.F:
                self._wait(pending_f.pop((action.stage, mb), ()), action)
                t0 = timer.start() if timer else None
                with record_function(f"Forward {mb}" if self._num_local == 1 else f"Stage {action.stage} Forward {mb}"):
                    if st.is_first:
                        out = st.forward_one_chunk(mb, arg_mbs[mb], kwarg_mbs[mb])
                    else:
                        out = st.forward_one_chunk(mb, (), {})
                    out_tuple = out if isinstance(out, tuple) else (out,)
                    for out_idx, dst in st.local_forward_targets():
                        stages[dst].set_local_input(mb, st.stage_index, out_idx, out_tuple[out_idx])
                    self._maybe_compute_loss(st, out, target_mbs, mb)
                if timer:
                    timer.stop(action, t0)
            elif op in (Op.B, Op.I):
                self._wait(pending_b.pop((action.stage, mb), ()), action)
                t0 = timer.start() if timer else None
                with record_function(f"Backward {mb}" if self._num_local == 1 else f"Stage {action.stage} Backward {mb}"):
                    st._configure_data_parallel_mode(self._last_backward_mb.get(action.stage) == mb)
                    loss = self._maybe_get_loss(st, mb)
                    st.backward_one_chunk(mb, loss=loss, full_backward=(op == Op.B))
                    grads = st.grads_input[mb]
                    for idx, spec in enumerate(st.input_specs):
                        if spec.source is not None and st.is_local_stage(spec.source):
                            stages[spec.source].set_local_out_grad(mb, spec.source_output, st.stage_index, grads[idx])
                if timer:
                    timer.stop(action, t0)
            elif op == Op.W:
                t0 = timer.start() if timer else None
                with record_function(f"Stage {action.stage} Weight {mb}"):
                    st.backward_weight_one_chunk(mb)
                if timer:
                    timer.stop(action, t0)
            elif op == Op.REDUCE_GRAD:
                if self.grad_reducer is not None:
                    self.grad_reducer.reduce_stage(st)
            else:  # pragma: no cover
                raise RuntimeError(f"unknown action {action}")

        self._wait(send_works, Action(self._stages[0].stage_index, Op.SEND_F))
        # the reducer's kernels run on a side stream over the same flat gradient buffer: this stream must wait for
        # them before anything else (the scaling below, the optimizer) touches the gradients
        if self.grad_reducer is not None and self._has_backward:
            self.grad_reducer.finish()
        if self.grad_reducer is not None and hasattr(self.grad_reducer, "check_read"):
            self.grad_reducer.check_read()  # debug mode (PIPPY_STREAM_CHECK=1): fails if a reduction is still in flight
        if self.scale_grads and self._has_backward:
            for st in self._stages:
                st.scale_grads(self._n_microbatches)
        if timer:
            timer.end_step()
            self.last_step_stats = timer.summary()
        self._update_losses(losses)

    # ------------------------------------------------------------------ public
    def step(self, *args, target=None, losses: Optional[List] = None, **kwargs):
        """Runs one full batch through the pipeline.

        The rank holding the first stage passes the model inputs, the rank holding the last stage passes
        ``target`` (when a loss function is set) and may pass a ``losses`` list to receive the per-microbatch
        losses; it gets the merged output back. Every other rank calls ``step()`` and gets ``None``.
        """
        for st in self._stages:
            st.clear_runtime_states()
            st.has_backward = self._has_backward
            st.keep_outputs = self.return_outputs
        args_split, kwargs_split = self._split_inputs(args, kwargs)
        if target is not None:
            targets_split = list(torch.tensor_split(target, self._n_microbatches))
        else:
            targets_split = None
        self._step_microbatches(args_split, kwargs_split, targets_split, losses)
        if not self.return_outputs:
            return None
        for st in self._stages:
            if st.is_last:
                chunks = [st.output_chunks[mb] for mb in range(self._n_microbatches)]
                return self._merge_outputs(chunks)
        return None


class PipelineScheduleSingle(PipelineSchedule):
    """Schedules with one stage per rank."""

    def __init__(self, stage: PipelineStageBase, n_microbatches: int, loss_fn=None, output_merge_spec=None, **kw):
        if isinstance(stage, (list, tuple)):
            if len(stage) != 1:
                raise ValueError(f"{type(self).__name__} takes exactly one stage per rank, got {len(stage)}")
            stage = stage[0]
        super().__init__([stage], n_microbatches, loss_fn, output_merge_spec, **kw)
        self._stage = stage
        if stage.num_stages != self.pp_group_size:
            raise ValueError(
                f"{type(self).__name__} runs one stage per rank: {stage.num_stages} stages need {stage.num_stages} "
                f"ranks but the pipeline group has {self.pp_group_size}"
            )


class ScheduleGPipe(PipelineScheduleSingle):
    """Fill-drain: all forwards, then all backwards."""

    def _compute_order(self) -> Schedule:
        return generators.gpipe(self.pp_group_size, self._n_microbatches, self._has_backward)


class Schedule1F1B(PipelineScheduleSingle):
    """One-forward-one-backward. ``reference_warmup=True`` reproduces the reference's deeper warm-up."""

    def __init__(self, stage, n_microbatches, loss_fn=None, output_merge_spec=None, reference_warmup=False, **kw):
        super().__init__(stage, n_microbatches, loss_fn, output_merge_spec, **kw)
        self.reference_warmup = reference_warmup

    def _compute_order(self) -> Schedule:
        return generators.one_f_one_b(
            self.pp_group_size, self._n_microbatches, self._has_backward, self.reference_warmup
        )


class PipelineScheduleMulti(PipelineSchedule):
    """Schedules with several stages per rank (stage ``rank + k * group_size``)."""

    _min_local_stages = 2

    def __init__(self, stages: List[PipelineStageBase], n_microbatches: int, loss_fn=None, output_merge_spec=None, **kw):
        if isinstance(stages, PipelineStageBase):
            stages = [stages]
        if len(stages) < self._min_local_stages:
            raise ValueError(
                f"{type(self).__name__} needs at least {self._min_local_stages} stages per rank, got {len(stages)}"
            )
        super().__init__(stages, n_microbatches, loss_fn, output_merge_spec, **kw)
        expected = [self.rank + k * self.pp_group_size for k in range(len(stages))]
        got = [s.stage_index for s in self._stages]
        if got != expected:
            raise ValueError(f"rank {self.rank} must hold stages {expected} for interleaving, got {got}")
        if self.num_stages != self.pp_group_size * len(stages):
            raise ValueError(
                f"{self.num_stages} stages cannot be spread as {len(stages)} per rank over {self.pp_group_size} ranks"
            )


class ScheduleLoopedBFS(PipelineScheduleMulti):
    """Breadth-first: every microbatch through one local stage before the next."""

    def _compute_order(self) -> Schedule:
        return generators.looped_bfs(self.pp_group_size, self._num_local, self._n_microbatches, self._has_backward)


class ScheduleInterleaved1F1B(PipelineScheduleMulti):
    """Interleaved 1F1B over ``v`` local stages; needs ``n_microbatches % pp_group_size == 0``."""

    def __init__(self, stages, n_microbatches, loss_fn=None, output_merge_spec=None, **kw):
        super().__init__(stages, n_microbatches, loss_fn, output_merge_spec, **kw)
        if n_microbatches % self.pp_group_size != 0:
            raise ValueError(
                f"Interleaved 1F1B requires the number of microbatches ({n_microbatches}) to be a multiple of the "
                f"pipeline group size ({self.pp_group_size})"
            )

    def _compute_order(self) -> Schedule:
        return generators.interleaved_1f1b(
            self.pp_group_size, self._num_local, self._n_microbatches, self._has_backward
        )


class ScheduleInterleavedZeroBubble(PipelineScheduleMulti):
    """Zero-bubble schedule: backward split into input-gradient (I) and weight-gradient (W) passes, W fills the
    gaps. Works with one or more stages per rank."""

    _min_local_stages = 1

    def __init__(self, stages, n_microbatches, loss_fn=None, output_merge_spec=None, max_pending_w=None,
                 extra_in_flight=0, **kw):
        super().__init__(stages, n_microbatches, loss_fn, output_merge_spec, **kw)
        self.max_pending_w = max_pending_w
        self.extra_in_flight = extra_in_flight
        self.stage_costs: Optional[Dict[int, Tuple[float, float, float]]] = None
        self.comm_latency = 0.0
        # how many microbatches beyond the 1F1B depth the cost-aware order may keep in flight per rank (each costs
        # one stage's activations); deep pipelines need several to cover the round trip of the first gradient
        self.max_extra_in_flight = 2
        if self._num_local > 1 and n_microbatches % self.pp_group_size != 0:
            raise ValueError(
                f"interleaved zero-bubble requires the number of microbatches ({n_microbatches}) to be a multiple of "
                f"the pipeline group size ({self.pp_group_size})"
            )

    def _compute_order(self) -> Schedule:
        if not self._has_backward:
            return generators.interleaved_1f1b(self.pp_group_size, self._num_local, self._n_microbatches, False)
        if self.stage_costs is not None:
            extras = tuple(e for e in (0, 1, 2, 4, 6, 8, 12, 16) if e <= self.max_extra_in_flight)
            return generators.tuned_zero_bubble_costed(
                self.pp_group_size, self._num_local, self._n_microbatches, self.stage_costs, self.comm_latency,
                extra_in_flight=extras,
                # parked weight-gradient passes hold their operands: never more of them than the default order parks
                pending_w=(self.pp_group_size, 2 * self.pp_group_size),
            )
        return generators.zero_bubble(
            self.pp_group_size, self._num_local, self._n_microbatches, self.max_pending_w, self.extra_in_flight
        )

    def set_stage_costs(self, costs: Dict[int, Tuple[float, float, float]], comm_latency: float = 0.0) -> None:
        """Rebuilds the order from measured costs: ``costs[s] = (forward, input-gradient, weight-gradient)`` seconds
        per microbatch for EVERY stage of the pipeline, identical on every rank (the order is derived from them
        deterministically, and all ranks must derive the same one)."""
        if sorted(costs) != list(range(self.num_stages)):
            raise ValueError(f"costs must cover stages 0..{self.num_stages - 1}")
        self.stage_costs = {int(s): tuple(float(x) for x in c) for s, c in costs.items()}
        self.comm_latency = ({int(k): float(v) for k, v in comm_latency.items()} if isinstance(comm_latency, dict)
                             else float(comm_latency))
        self._build()

    def retune_from_last_step(self, comm_latency=0.0, p2p_bytes_per_s: Optional[float] = None,
                              max_extra_in_flight: Optional[int] = None):
        """Collective over the pipeline group: gathers every rank's measured per-stage F / I / W means of the last
        step (which must have run with ``record_timing``) and rebuilds the order from them.  With
        ``p2p_bytes_per_s`` the transfer time of every stage boundary is derived from the bytes the producing stage
        sends (boundaries inside a layer carry two tensors) instead of one ``comm_latency`` for all."""
        if self.last_step_stats is None:
            raise RuntimeError("run one step with record_timing=True first")
        mine = dict(self.last_step_stats["per_stage_op_mean_s"])
        for st in self._stages:
            nbytes = sum(m.shape.numel() * torch.empty((), dtype=m.dtype).element_size() for m in st.output_metas)
            mine[f"{st.stage_index}:bytes"] = float(nbytes)
        tables: List[Optional[dict]] = [None] * self.pp_group_size
        if self.pp_group_size > 1:
            dist.all_gather_object(tables, mine, group=self._stages[0].group)
        else:
            tables = [mine]
        merged: Dict[str, float] = {}
        for t in tables:
            merged.update(t)
        costs = {}
        for s in range(self.num_stages):
            f, i, w = merged.get(f"{s}:F"), merged.get(f"{s}:I"), merged.get(f"{s}:W")
            if f is None or i is None or w is None:
                raise RuntimeError(f"no measured F / I / W time for stage {s}: the last step did not run a split backward")
            costs[s] = (f, i, w)
        if p2p_bytes_per_s:
            comm_latency = {s: merged.get(f"{s}:bytes", 0.0) / p2p_bytes_per_s for s in range(self.num_stages - 1)}
        if max_extra_in_flight is not None:
            self.max_extra_in_flight = int(max_extra_in_flight)  # must be the same on every rank
        self.set_stage_costs(costs, comm_latency)
        return costs


ScheduleZeroBubble = ScheduleInterleavedZeroBubble


class ScheduleZBVZeroBubble(PipelineSchedule):
    """Zero-bubble schedule on the V-shaped placement: rank r holds stage r and stage 2P-1-r, so the first and the
    last stage (embedding and LM head, a tied pair in many models) share rank 0 and the turn of the V is a local
    hand-over.  Upstream's ScheduleZBVZeroBubble (torch/distributed/pipelining/schedules.py:2811-3000) hard-codes
    its order; here the order comes from list scheduling on the cost model (``generators.tuned_zero_bubble_placed``).
    The stages' placement is set by this constructor."""

    def __init__(self, stages, n_microbatches, loss_fn=None, output_merge_spec=None, cost_f=2, cost_i=3, cost_w=2, **kw):
        stages = list(stages)
        if len(stages) != 2:
            raise ValueError(f"ScheduleZBVZeroBubble needs exactly 2 stages per rank, got {len(stages)}")
        first = min(stages, key=lambda s: s.stage_index)
        P = first.group_size
        placement = generators.v_placement(P)
        expected = sorted(s for s, r in placement.items() if r == first.group_rank)
        got = sorted(s.stage_index for s in stages)
        if first.num_stages != 2 * P or got != expected:
            raise ValueError(f"rank {first.group_rank} must hold stages {expected} of {2 * P} for the V shape, got {got}")
        for st in stages:
            st.set_placement(placement)
        self._costs = (cost_f, cost_i, cost_w)
        super().__init__(stages, n_microbatches, loss_fn, output_merge_spec, **kw)

    def _compute_order(self) -> Schedule:
        placement = self._stages[0].stage_index_to_group_rank
        if not self._has_backward:
            # forward only: every rank runs its stages' forwards in dependency order, nearest the loss first
            order = generators.zero_bubble_placed(self.pp_group_size, placement, self._n_microbatches)
            return {r: [a for a in acts if a.op == Op.F] for r, acts in order.items()}
        return generators.tuned_zero_bubble_placed(self.pp_group_size, placement, self._n_microbatches, *self._costs)
