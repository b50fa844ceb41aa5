"""Stages built from a hand-written ``nn.Module`` plus example tensors, no tracing
(reference pippy/ManualPipelineStage.py).

Topology is a chain: every input comes from stage ``i-1`` and every output goes to stage ``i+1``.
Also here: the shape metadata exchange used to check that neighbouring stages agree
(``get_stage_shapes`` :105-175, ``validate_stage_shapes`` :342-439 in the reference).
"""
from __future__ import annotations

import logging
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn

from .stage import InputSpec, PipelineStageBase, TensorMeta

logger = logging.getLogger("pippy_b200")

METADATA_TENSOR_LEN = 100
PLACEHOLDER_VAL = -1

_DTYPE_CODES = [
    torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int32, torch.int16, torch.int8,
    torch.uint8, torch.bool,
]


def _as_tensor_list(value, what: str) -> List[torch.Tensor]:
    if isinstance(value, torch.Tensor):
        return [value]
    if isinstance(value, (tuple, list)):
        for v in value:
            if not isinstance(v, torch.Tensor):
                raise TypeError(f"Unsupported type {type(v)} in {what}: cannot create empty tensors")
        return list(value)
    raise TypeError(f"Unsupported type {type(value)} for {what}: cannot create empty tensors")


def create_empty_tensors(tensors, device: torch.device) -> List[torch.Tensor]:
    """Empty tensors with the shapes/dtypes of ``tensors`` on ``device`` (tensors may live on ``meta``)."""
    return [torch.empty(t.shape, dtype=t.dtype, device=device) for t in _as_tensor_list(tensors, "stage arguments")]


def create_metadata_tensor(
    tensors: Optional[Sequence[torch.Tensor]] = None, device: Union[torch.device, str] = "cpu"
) -> torch.Tensor:
    """Encodes the shapes of up to a few tensors in a fixed int32[100]: ``[ndim, d0, d1, ...]`` per tensor,
    padded with -1.  Raises ValueError when they do not fit."""
    md = torch.full((METADATA_TENSOR_LEN,), PLACEHOLDER_VAL, dtype=torch.int32, device=device)
    if tensors:
        data: List[int] = []
        for t in tensors:
            data.append(t.dim())
            data.extend(t.shape)
        if len(data) > METADATA_TENSOR_LEN:
            raise ValueError(
                f"Metadata of the tensors needs {len(data)} entries, more than the {METADATA_TENSOR_LEN} available"
            )
        md[: len(data)] = torch.tensor(data, dtype=torch.int32, device=device)
    return md


def extract_metadata_from_tensor(md: torch.Tensor) -> List[torch.Size]:
    values = md.tolist()
    shapes: List[torch.Size] = []
    i = 0
    while i < len(values) and values[i] != PLACEHOLDER_VAL:
        ndim = values[i]
        shapes.append(torch.Size(values[i + 1 : i + 1 + ndim]))
        i += 1 + ndim
    return shapes


class ManualPipelineStage(PipelineStageBase):
    """A pipeline stage around a user-supplied module.

    ``input_args`` are example inputs (only shape/dtype matter; ``meta`` tensors are fine). When
    ``output_args`` is omitted the module is run once on empty inputs to find the output shapes.
    """

    def __init__(
        self,
        submodule: nn.Module,
        stage_index: int,
        num_stages: int,
        device: torch.device,
        num_microbatches: int,
        input_args: Union[torch.Tensor, Sequence[torch.Tensor]],
        output_args: Optional[Union[torch.Tensor, Sequence[torch.Tensor]]] = None,
        group: Optional[dist.ProcessGroup] = None,
    ):
        super().__init__(submodule, stage_index, num_stages, device, group)
        inputs = _as_tensor_list(input_args, "input_args")
        if output_args is None:
            run_device = inputs[0].device if inputs and inputs[0].device.type == "meta" else self.device
            probe = [torch.empty(t.shape, dtype=t.dtype, device=run_device) for t in inputs]
            with torch.no_grad():
                out = submodule(*probe)
            outputs = _as_tensor_list(out, "the stage module's output")
        else:
            outputs = _as_tensor_list(output_args, "output_args")
        self.inputs_meta = [TensorMeta.of(t) for t in inputs]
        self.output_metas = [TensorMeta.of(t) for t in outputs]
        self.input_specs = [
            InputSpec(f"input{i}", None if self.is_first else stage_index - 1, i, m)
            for i, m in enumerate(self.inputs_meta)
        ]
        self.output_dests = {i: ([] if self.is_last else [stage_index + 1]) for i in range(len(outputs))}
        self.prev_stage = (self.group_rank - 1) % self.group_size
        self.next_stage = (self.group_rank + 1) % self.group_size
        self._prepare_forward_infra(num_microbatches)
        logger.debug(
            "[%d] manual stage: inputs %s outputs %s", stage_index,
            [tuple(m.shape) for m in self.inputs_meta], [tuple(m.shape) for m in self.output_metas],
        )

    def init_p2p_neighbors(self) -> bool:
        """Exchanges one element with both neighbours so the transport sets up its connections before the first
        step (the reference builds these ops, pippy/ManualPipelineStage.py:309-339, but never issues them)."""
        if not dist.is_initialized() or self.group_size == 1:
            return True
        ops = []
        recv_next = torch.zeros(1, device=self.device)
        recv_prev = torch.zeros(1, device=self.device)
        send = torch.ones(1, device=self.device)
        if not self.is_first and not self.is_local_stage(self.stage_index - 1):
            prev = self._global_rank(self.rank_of_stage(self.stage_index - 1))
            ops.append(dist.P2POp(dist.irecv, recv_prev, prev, self.group))
            ops.append(dist.P2POp(dist.isend, send, prev, self.group))
        if not self.is_last and not self.is_local_stage(self.stage_index + 1):
            nxt = self._global_rank(self.rank_of_stage(self.stage_index + 1))
            ops.append(dist.P2POp(dist.isend, send, nxt, self.group))
            ops.append(dist.P2POp(dist.irecv, recv_next, nxt, self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return True


def get_stage_shapes(
    stage_modules: List[nn.Module],
    stage_ids: List[int],
    num_stages: int,
    rank: int,
    world_size: int,
    device: torch.device,
    microbatch: Optional[Union[torch.Tensor, Sequence[torch.Tensor]]] = None,
    group: Optional[dist.ProcessGroup] = None,
    dtype: Optional[torch.dtype] = None,
) -> Dict[int, Dict[str, List[torch.Size]]]:
    """Dry-runs the pipeline once to learn every local stage's input and output shapes.

    Ranks proceed in stage order: receive the input shapes from the previous stage's rank, run the module on empty
    tensors, send the output shapes on.  Returns ``{stage_id: {"inputs": [...], "outputs": [...]}}``.
    ``dtype`` is the dtype of the probe tensors of non-first stages (default: the module's first parameter's).
    """
    shapes: Dict[int, Dict[str, List[torch.Size]]] = {}
    for module, stage_id in zip(stage_modules, stage_ids):
        if stage_id == 0:
            if microbatch is None:
                raise RuntimeError("Microbatch is required for first stage")
            example = _as_tensor_list(microbatch, "microbatch")
            input_shapes = [t.shape for t in example]
            probe = [torch.empty(t.shape, dtype=t.dtype, device=device) for t in example]
        else:
            md = create_metadata_tensor(device=device)
            prev_rank = (stage_id - 1) % world_size
            if prev_rank == rank:
                input_shapes = shapes[stage_id - 1]["outputs"]
            else:
                src = prev_rank if group is None else dist.get_global_rank(group, prev_rank)
                dist.recv(md, src=src, group=group)
                input_shapes = extract_metadata_from_tensor(md)
            probe_dtype = dtype
            if probe_dtype is None:
                first = next(module.parameters(), None)
                probe_dtype = first.dtype if first is not None else torch.get_default_dtype()
            probe = [torch.empty(s, dtype=probe_dtype, device=device) for s in input_shapes]
        with torch.no_grad():
            out = module(*probe)
        outs = _as_tensor_list(out, "the stage module's output")
        output_shapes = [t.shape for t in outs]
        shapes[stage_id] = {"inputs": list(input_shapes), "outputs": output_shapes}
        if stage_id != num_stages - 1:
            next_rank = (stage_id + 1) % world_size
            if next_rank != rank:
                dst = next_rank if group is None else dist.get_global_rank(group, next_rank)
                dist.send(create_metadata_tensor(outs, device=device), dst=dst, group=group)
    return shapes


def validate_stage_shapes(pipeline_stages: List[ManualPipelineStage]) -> None:
    """All-gathers every stage's input/output shapes and checks outputs of stage i equal inputs of i+1."""
    if len(pipeline_stages) == 0:
        raise ValueError("No pipeline stages provided.")
    virtual = len(pipeline_stages)
    first = pipeline_stages[0]
    all_inputs, all_outputs = [], []
    world_size = first.group_size
    num_stages = first.num_stages
    for st in pipeline_stages:
        if st.group_size != world_size:
            raise ValueError(f"Stage {st.stage_index} has group size {st.group_size}, expected {world_size}")
        if st.num_stages != num_stages:
            raise ValueError(f"Stage {st.stage_index} has num_stages {st.num_stages}, expected {num_stages}")
        if st.group_rank != first.group_rank:
            raise ValueError(f"Stage {st.stage_index} has rank {st.group_rank}, expected {first.group_rank}")
    if num_stages % world_size != 0:
        raise ValueError(f"Number of stages {num_stages} must be a multiple of the world size {world_size}")
    for st in pipeline_stages:
        in_md = create_metadata_tensor([torch.empty(m.shape, device="meta") for m in st.inputs_meta], device=st.device)
        out_md = create_metadata_tensor([torch.empty(m.shape, device="meta") for m in st.output_metas], device=st.device)
        gathered_in = [torch.empty_like(in_md) for _ in range(world_size)]
        gathered_out = [torch.empty_like(out_md) for _ in range(world_size)]
        if dist.is_initialized() and world_size > 1:
            dist.all_gather(gathered_in, in_md, group=st.group)
            dist.all_gather(gathered_out, out_md, group=st.group)
        else:
            gathered_in, gathered_out = [in_md], [out_md]
        all_inputs.extend(extract_metadata_from_tensor(t) for t in gathered_in)
        all_outputs.extend(extract_metadata_from_tensor(t) for t in gathered_out)
    # entry k*world + r describes stage (k*world + r)
    for i in range(virtual * world_size - 1):
        if all_outputs[i] != all_inputs[i + 1]:
            raise ValueError(
                f"Stage {i} output shapes {all_outputs[i]} do not match stage {i + 1} input shapes {all_inputs[i + 1]}"
            )
