"""Runtime stage backed by a traced :class:`~pippy_b200.ir.Pipe`
(reference pippy/_PipelineStage.py:553-833).

The stage's wiring is read off the split program: which model inputs or which outputs of earlier stages feed each
placeholder of the stage module, and which later stages consume each of its outputs.  A value may fan out to
several stages (skip connections); gradients of such a value are summed when they come back, which the reference
asserts out (pippy/_PipelineStage.py:799-802).
"""
from __future__ import annotations

import logging
import operator
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.fx as fx

from .ir import Pipe
from .stage import InputSpec, PipelineStageBase, RecvInfo, TensorMeta
from .utils.graph import modify_graph_op_device

logger = logging.getLogger("pippy_b200")


def _meta_of(node: fx.Node) -> Optional[TensorMeta]:
    val = node.meta.get("val") if isinstance(node, fx.Node) else None
    if isinstance(val, torch.Tensor):
        return TensorMeta(torch.Size(val.shape), val.dtype)
    return None


class PipelineStage(PipelineStageBase):
    def __init__(self, pipe: Pipe, stage_index: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        submod = pipe.get_stage_module(stage_index)
        self.pipe = pipe
        self.pipe_info = pipe.info()
        super().__init__(submod, stage_index, self.pipe_info.num_stages, device, group)
        graph = pipe.split_gm.graph
        calls = [n for n in graph.nodes if n.op == "call_module"]
        if len(calls) != self.num_stages:
            raise AssertionError(
                f"Number of submodules in pipe graph {len(calls)} does not match number of stages {self.num_stages}"
            )
        self.submod_to_stage_index: Dict[str, int] = {str(n.target): i for i, n in enumerate(calls)}
        self.node = calls[stage_index]
        placeholders_root = [n for n in graph.nodes if n.op == "placeholder"]
        self._root_index = {n: i for i, n in enumerate(placeholders_root)}

        # ---- inputs
        sub_placeholders = [n for n in submod.graph.nodes if n.op == "placeholder"]
        self.input_specs = []
        self._root_arg_index: List[Optional[int]] = []
        for ph, arg in zip(sub_placeholders, self.node.args):
            src_stage, src_out = self._producer(arg)
            meta = _meta_of(ph)
            self.input_specs.append(InputSpec(ph.name, src_stage, src_out, meta))
            self._root_arg_index.append(self._root_index.get(arg) if src_stage is None else None)

        # ---- outputs
        out_node = next(n for n in submod.graph.nodes if n.op == "output")
        outs = out_node.args[0]
        outs = list(outs) if isinstance(outs, (tuple, list)) else [outs]
        self.output_metas = [(_meta_of(o) or TensorMeta(torch.Size([]), torch.float32)) for o in outs]
        self.output_dests = {i: [] for i in range(len(outs))}
        for user in self.node.users:
            if user.op == "call_function" and user.target is operator.getitem:
                idx = user.args[1]
                for uu in user.users:
                    if uu.op == "call_module":
                        self.output_dests[idx].append(self.submod_to_stage_index[str(uu.target)])
            elif user.op == "call_module":
                self.output_dests[0].append(self.submod_to_stage_index[str(user.target)])
        for k in self.output_dests:
            self.output_dests[k] = sorted(set(self.output_dests[k]))

        # ---- topology of the whole pipeline, for the schedule's communication planning
        self.global_dests: Dict[int, List[int]] = {i: [] for i in range(self.num_stages)}
        for i, call in enumerate(calls):
            consumers = set()
            for user in call.users:
                if user.op == "call_function" and user.target is operator.getitem:
                    consumers.update(self.submod_to_stage_index[str(uu.target)] for uu in user.users if uu.op == "call_module")
                elif user.op == "call_module":
                    consumers.add(self.submod_to_stage_index[str(user.target)])
            self.global_dests[i] = sorted(consumers)

        self._move_submod_to_device()
        modify_graph_op_device(self.submod, self.device)
        if self.pipe_info.num_chunks is not None:
            self._prepare_forward_infra(self.pipe_info.num_chunks)

    def _producer(self, arg) -> Tuple[Optional[int], int]:
        if not isinstance(arg, fx.Node):
            return None, 0
        if arg.op == "call_module":
            return self.submod_to_stage_index[str(arg.target)], 0
        if arg.op == "call_function" and arg.target is operator.getitem and isinstance(arg.args[0], fx.Node) \
                and arg.args[0].op == "call_module":
            return self.submod_to_stage_index[str(arg.args[0].target)], int(arg.args[1])
        return None, 0

    def _move_submod_to_device(self) -> None:
        has_meta = any(
            isinstance(p, torch._subclasses.FakeTensor) or p.is_meta for p in self.submod.parameters()
        )
        if has_meta:
            logger.debug("[%d] stage module has meta parameters; leaving it for the user to materialise", self.stage_index)
        else:
            self.submod.to(self.device)

    # model inputs arrive as the caller's (args, kwargs); map them to this stage's placeholders
    def _compose_inputs(self, mb: int, args: Tuple[Any, ...], kwargs: Optional[Dict[str, Any]] = None) -> List[Any]:
        infos = self.args_recv_info[mb]
        flat_root: Optional[List[Any]] = None
        local = self.local_inputs.get(mb, {})
        composite: List[Any] = []
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
                if flat_root is None:
                    if not args and not kwargs:
                        raise RuntimeError(
                            f"[{self.stage_index}] needs model input {spec.name!r}; pass the model inputs to step() on "
                            "this rank"
                        )
                    flat_root = self.pipe.flatten_inputs(tuple(args), dict(kwargs or {}))
                composite.append(flat_root[self._root_arg_index[idx]])
        return composite

    def forward_one_chunk(self, *call_args, **call_kwargs):
        mb, args, kwargs = self._parse_chunk_call(call_args, call_kwargs, forward=True)
        self._pending_kwargs = kwargs
        try:
            return super().forward_one_chunk(mb, args, {})
        finally:
            self._pending_kwargs = None

    def _compose_inputs_base(self, mb, args):  # pragma: no cover - kept for clarity
        return super()._compose_inputs(mb, args)


# route the base class's composition through the traced variant (which also sees the keyword inputs)
def _compose_dispatch(self, mb, args):
    return PipelineStage._compose_inputs(self, mb, args, getattr(self, "_pending_kwargs", None))


PipelineStage._compose_inputs_for_forward = _compose_dispatch
