"""Tracing front-end: turns an unmodified ``nn.Module`` into a :class:`Pipe` of stage modules.

Public surface follows the reference (pippy/_IR.py): ``pipe_split()``, ``SplitPoint``, ``annotate_split_points``,
``pipeline()``, ``Pipe`` (``num_stages``, ``get_stage_module``, ``info``, ``split_gm``, ``replicated_params``,
local execution by calling the pipe), ``ArgsChunkSpec`` / ``KwargsChunkSpec``, ``MultiUseParameterConfig``,
``LossWrapper`` / ``TrivialLossWrapper``, ``PipeSequential``.

How a model is split (own implementation; nothing is vendored from torch internals):
  1. ``torch.export`` of one microbatch gives a flat ATen graph in which the ``pipe_split`` marker op survives;
  2. guard bookkeeping nodes are dropped, redundant markers collapsed, ``fx.passes.split_module`` cuts at markers;
  3. every parameter/buffer a partition uses is re-homed inside that partition under its ORIGINAL qualified name
     (intermediate containers are created on the way), so the union of the stages' ``state_dict()`` keys equals
     the model's own key set;
  4. a tensor used by several stages (tied weights) is either replicated (each later stage gets its own copy and the
     group is recorded in ``Pipe.replicated_params`` so the runtime can sum the gradients) or transmitted (it stays
     on its first stage and travels as an extra stage output).  The reference raises NotImplementedError here
     (pippy/_IR.py:871-879).
"""
from __future__ import annotations

import copy
import inspect
import logging
import operator
from dataclasses import dataclass
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import torch
import torch.fx as fx
import torch.nn as nn
from torch.fx.passes.split_module import split_module
from torch.utils import _pytree as pytree

from .backward import _null_coalesce_accumulate, stage_backward
from .microbatch import TensorChunkSpec, split_args_kwargs_into_chunks

logger = logging.getLogger("pippy_b200")

# ------------------------------------------------------------------------------------------------
# the marker op
# ------------------------------------------------------------------------------------------------
_LIB = torch.library.Library("pippy_b200", "DEF")
_LIB.define("_pipe_split() -> ()")


@torch.library.impl(_LIB, "_pipe_split", "BackendSelect")
def _pipe_split_impl():
    return None


@torch.library.register_fake("pippy_b200::_pipe_split")
def _pipe_split_fake():
    return None


# dead-code elimination must keep the marker
fx.node._side_effectful_functions.add(torch.ops.pippy_b200._pipe_split.default)
fx.node._side_effectful_functions.add(torch.ops.pippy_b200._pipe_split)

aten_pipe_split_alias = torch.ops.pippy_b200._pipe_split.default


def pipe_split() -> None:
    """Marks a stage boundary. A no-op when the model runs eagerly; the splitter cuts the traced graph here."""
    return torch.ops.pippy_b200._pipe_split()


def _is_split(node: fx.Node) -> bool:
    return node.op == "call_function" and node.target in (
        torch.ops.pippy_b200._pipe_split.default,
        torch.ops.pippy_b200._pipe_split,
    )


class SplitPoint(Enum):
    BEGINNING = 1
    END = 2


class PipeSplitWrapper:
    """Kept for scripts written against the older spelling ``PipeSplitWrapper.SplitPoint``."""

    SplitPoint = SplitPoint


def annotate_split_points(mod: nn.Module, spec: Dict[str, SplitPoint]) -> None:
    """Patches the ``forward`` of each named submodule so that it calls :func:`pipe_split` before
    (``BEGINNING``) or after (``END``) running. The module is modified in place."""
    for qualname, split_type in spec.items():
        atoms = qualname.split(".")
        target = mod
        for i, atom in enumerate(atoms):
            try:
                target = getattr(target, atom)
            except AttributeError as e:
                raise AttributeError(
                    f'Specified target {qualname} referenced nonexistent module {".".join(atoms[: i + 1])}'
                ) from e
        if split_type not in (SplitPoint.BEGINNING, SplitPoint.END):
            raise ValueError("Unknown split point type.")
        _patch_forward(target, split_type)


def _patch_forward(target: nn.Module, split_type: SplitPoint) -> None:
    original = target.forward

    if split_type == SplitPoint.BEGINNING:

        def forward(*args, **kwargs):
            pipe_split()
            return original(*args, **kwargs)

    else:

        def forward(*args, **kwargs):
            try:
                return original(*args, **kwargs)
            finally:
                pipe_split()

    target.forward = forward
    target._pb_original_forward = original


class MultiUseParameterConfig(Enum):
    TRANSMIT = 1
    REPLICATE = 2


MultiUseParamSpec = Union[MultiUseParameterConfig, Dict[str, MultiUseParameterConfig]]


# ------------------------------------------------------------------------------------------------
# loss wrappers (for models whose forward computes the loss)
# ------------------------------------------------------------------------------------------------
class LossWrapper(nn.Module):
    """Base class for wrapping a module and a loss function so the traced program returns the loss
    (reference _IR.py:36-120). Subclasses define ``forward(self, input, target)``."""

    def __init__(self, module: nn.Module, loss_fn: Callable):
        super().__init__()
        self.module = module
        self.loss_fn = loss_fn

    def forward(self, *args, **kwargs):
        raise NotImplementedError("Subclasses of LossWrapper define forward(input..., target) and return the loss")


class TrivialLossWrapper(LossWrapper):
    loss_spec = True

    def forward(self, x, targets):
        return self.loss_fn(self.module(x), targets)


class PipeSequential(nn.Sequential):
    """``nn.Sequential`` that marks a stage boundary between consecutive children."""

    @staticmethod
    def from_sequential(seq: nn.Sequential) -> "PipeSequential":
        return PipeSequential(*[copy.copy(m) for m in seq])

    def forward(self, x):
        for i, module in enumerate(self):
            x = module(x)
            if i != len(self) - 1:
                pipe_split()
        return x


# ------------------------------------------------------------------------------------------------
# local executor
# ------------------------------------------------------------------------------------------------
class DetachExecutor(fx.Interpreter):
    """Runs the split program in one process the way the distributed runtime would: every tensor that crosses into
    a stage is detached first, so each stage is its own autograd island (reference _IR.py:355-404)."""

    def __init__(self, module, garbage_collect_values=True):
        garbage_collect_values = False
        super().__init__(module, garbage_collect_values)
        self.value_remap: Dict[int, torch.Tensor] = {}

    def _detach(self, a):
        if isinstance(a, torch.Tensor) and a.requires_grad and not isinstance(a, nn.Parameter):
            key = id(a)
            if key not in self.value_remap:
                self.value_remap[key] = a.detach().requires_grad_(True)
            return self.value_remap[key]
        return a

    def call_module(self, target, args, kwargs):
        args = pytree.tree_map(self._detach, args)
        kwargs = pytree.tree_map(self._detach, kwargs)
        return super().call_module(target, args, kwargs)

    def call_function(self, target, args, kwargs):
        if target is stage_backward:
            kwargs = dict(kwargs)
            kwargs["input_values"] = [self.value_remap.get(id(v), v) for v in kwargs["input_values"]]
        return super().call_function(target, args, kwargs)


# ------------------------------------------------------------------------------------------------
# Pipe
# ------------------------------------------------------------------------------------------------
@dataclass
class PipeInfo:
    graph: fx.Graph
    num_stages: int
    num_chunks: Optional[int]
    has_loss_and_backward: bool
    args_chunk_spec: Optional[Tuple[Any, ...]] = None
    kwargs_chunk_spec: Optional[Dict[str, Any]] = None


_ALLOWED_TOP_LEVEL = {"placeholder", "output", "call_module", "get_attr"}


def _assign_by_qualname(root: nn.Module, qualname: str, value, kind: str, persistent: bool = True) -> None:
    """Installs ``value`` at ``root.<qualname>`` creating empty container modules on the way."""
    *path, leaf = qualname.split(".")
    mod = root
    for atom in path:
        child = getattr(mod, atom, None)
        if not isinstance(child, nn.Module):
            child = nn.Module()
            setattr(mod, atom, child)
        mod = child
    if kind == "parameter":
        mod.register_parameter(leaf, value)
    elif kind == "buffer":
        if leaf in mod._buffers:
            mod._buffers[leaf] = value
        else:
            mod.register_buffer(leaf, value, persistent=persistent)
    else:
        setattr(mod, leaf, value)


def _get_by_qualname(root: nn.Module, qualname: str):
    obj = root
    for atom in qualname.split("."):
        obj = getattr(obj, atom)
    return obj


class Pipe(nn.Module):
    """The split program: ``split_gm`` is a graph whose nodes are the stage modules ``submod_0 … submod_{n-1}``
    (plus ``getitem`` and, when a loss spec was given, ``stage_backward`` calls)."""

    # chunk specs set by the ArgsChunkSpec / KwargsChunkSpec context managers (reference _IR.py:502-507)
    args_chunk_spec: Optional[Tuple[Any, ...]] = None
    kwargs_chunk_spec: Optional[Dict[str, Any]] = None

    def __init__(
        self,
        split_gm: fx.GraphModule,
        num_stages: int,
        has_loss_and_backward: bool,
        loss_spec: Any,
        signature: Optional[inspect.Signature],
        in_spec: Optional[pytree.TreeSpec],
        n_trace_args: int,
        trace_kwarg_names: List[str],
        qualname_mapping: Optional[Dict[str, str]] = None,
    ):
        super().__init__()
        self.split_gm = split_gm
        self.num_stages = num_stages
        self.has_loss_and_backward = has_loss_and_backward
        self.loss_spec = loss_spec
        self._signature = signature
        self._in_spec = in_spec
        self._n_trace_args = n_trace_args
        self._trace_kwarg_names = trace_kwarg_names
        self.new_to_old_qualname_mapping = qualname_mapping or {}
        self.pipe_info: Optional[PipeInfo] = None

        for node in split_gm.graph.nodes:
            ok = node.op in _ALLOWED_TOP_LEVEL or (node.op, node.target) in (
                ("call_function", operator.getitem),
                ("call_function", stage_backward),
                ("call_function", _null_coalesce_accumulate),
            )
            if not ok:
                raise AssertionError(f"unexpected node in the split program: {node.format_node()}")

        # tensors shared between stage modules are de-aliased; each group is recorded
        self.replicated_params: List[Dict[str, str]] = self._dealias_shared_tensors()

        def poisoned_forward(*args, **kwargs):
            raise RuntimeError("To run pipeline locally, invoke the Pipe object directly, not `split_gm`")

        self.split_gm.forward = poisoned_forward
        self.executor = DetachExecutor(self.split_gm)

    # -- structure -----------------------------------------------------------------------------
    def _stage_names(self) -> List[str]:
        return [f"submod_{i}" for i in range(self.num_stages)]

    def _dealias_shared_tensors(self) -> List[Dict[str, str]]:
        seen: Dict[int, Tuple[str, str]] = {}
        groups: Dict[int, Dict[str, str]] = {}
        for name in self._stage_names():
            submod = getattr(self.split_gm, name)
            for qual, t in list(submod.named_parameters(remove_duplicate=False)):
                key = id(t)
                if key in seen and seen[key][0] != name:
                    groups.setdefault(key, {seen[key][0]: seen[key][1]})
                    if name in groups[key]:
                        continue  # alias inside the same stage (e.g. two names of one tensor)
                    groups[key][name] = qual
                elif key not in seen:
                    seen[key] = (name, qual)
        out: List[Dict[str, str]] = []
        for key, group in groups.items():
            first = True
            for name, qual in group.items():
                if first:
                    first = False
                    continue
                submod = getattr(self.split_gm, name)
                orig = _get_by_qualname(submod, qual)
                clone = nn.Parameter(orig.detach().clone(), requires_grad=orig.requires_grad)
                # every alias of this tensor inside the stage moves to the clone
                for q2, t2 in list(submod.named_parameters(remove_duplicate=False)):
                    if t2 is orig:
                        _assign_by_qualname(submod, q2, clone, "parameter")
            out.append(group)
        return out

    def get_stage_module(self, stage_idx: int) -> nn.Module:
        if stage_idx < 0 or stage_idx >= self.num_stages:
            raise ValueError(f"Invalid stage index {stage_idx}!")
        return getattr(self.split_gm, f"submod_{stage_idx}")

    def info(self) -> PipeInfo:
        if self.pipe_info is None:
            raise RuntimeError("Pipe info is not available. Please use the `pipeline` method to create the `Pipe` object.")
        return self.pipe_info

    def build_stage(self, stage_index: int, device: torch.device, group=None):
        """Creates the runtime stage for ``stage_index`` on ``device`` (the newer spelling of
        ``PipelineStage(pipe, stage_index, device, group)``)."""
        from .pipeline_stage import PipelineStage

        return PipelineStage(self, stage_index, device, group)

    def remap_qualname(self, qualname: str) -> str:
        """Maps ``split_gm.submod_i.<fqn>`` (or ``submod_i.<fqn>``) back to the original model's name."""
        name = qualname
        if name.startswith("split_gm."):
            name = name[len("split_gm."):]
        if name in self.new_to_old_qualname_mapping:
            return self.new_to_old_qualname_mapping[name]
        head, _, rest = name.partition(".")
        if head.startswith("submod_") and rest:
            return rest
        # longest known prefix from the right
        atoms = name.split(".")
        for cut in range(len(atoms) - 1, 0, -1):
            prefix = ".".join(atoms[:cut])
            if prefix in self.new_to_old_qualname_mapping:
                return ".".join([self.new_to_old_qualname_mapping[prefix]] + atoms[cut:])
        return name

    # -- execution -----------------------------------------------------------------------------
    def flatten_inputs(self, args: Tuple[Any, ...], kwargs: Dict[str, Any]) -> List[Any]:
        """Binds ``(args, kwargs)`` like the original ``forward`` would and returns the flat list of graph inputs."""
        if self._signature is not None:
            bound = self._signature.bind(*args, **kwargs)  # raises the usual TypeError texts
            arguments = dict(bound.arguments)
            names = list(self._signature.parameters)
            pos = []
            for n in names[: self._n_trace_args]:
                if n in arguments:
                    pos.append(arguments.pop(n))
            var_pos = [n for n, p in self._signature.parameters.items() if p.kind == p.VAR_POSITIONAL]
            for n in var_pos:
                pos.extend(arguments.pop(n, ()))
            var_kw = [n for n, p in self._signature.parameters.items() if p.kind == p.VAR_KEYWORD]
            kw: Dict[str, Any] = {}
            for n in var_kw:
                kw.update(arguments.pop(n, {}))
            kw.update(arguments)
            args, kwargs = tuple(pos), kw
        kwargs = {k: kwargs[k] for k in self._trace_kwarg_names if k in kwargs} | {
            k: v for k, v in kwargs.items() if k not in self._trace_kwarg_names
        }
        flat, spec = pytree.tree_flatten((tuple(args), dict(kwargs)))
        if self._in_spec is not None and spec != self._in_spec:
            raise TypeError(
                "the arguments do not have the structure the model was traced with: "
                f"traced {self._in_spec}, got {spec}"
            )
        return flat

    def forward(self, *args, **kwargs):
        flat = self.flatten_inputs(args, kwargs)
        self.executor.value_remap = {}
        return self.executor.run(*flat)

    def print_readable(self) -> None:
        self.split_gm.print_readable()

    def __str__(self) -> str:
        return self.split_gm.__str__()

    def __repr__(self) -> str:
        return self.split_gm.__repr__()

    # -- construction --------------------------------------------------------------------------
    @staticmethod
    def _trace_with_export(mod: nn.Module, example_args, example_kwargs):
        logger.info("Tracing model with torch.export ...")
        return torch.export.export(mod, tuple(example_args), dict(example_kwargs or {}), strict=False)

    @staticmethod
    def from_tracing(
        mod: nn.Module,
        num_chunks: Optional[int],
        example_args: Tuple[Any, ...],
        example_kwargs: Optional[Dict[str, Any]] = None,
        split_policy: Optional[Callable[[fx.GraphModule], fx.GraphModule]] = None,
        multi_use_param_spec: MultiUseParamSpec = MultiUseParameterConfig.REPLICATE,
        output_loss_value_spec: Any = None,
        already_microbatch: bool = False,
    ) -> "Pipe":
        example_kwargs = example_kwargs or {}
        args_spec, kwargs_spec = Pipe.args_chunk_spec, Pipe.kwargs_chunk_spec
        if already_microbatch:
            mb_args, mb_kwargs = tuple(example_args), dict(example_kwargs)
        else:
            args_split, kwargs_split = split_args_kwargs_into_chunks(
                example_args, example_kwargs, num_chunks, args_spec, kwargs_spec
            )
            mb_args, mb_kwargs = args_split[0], kwargs_split[0]
        ep = Pipe._trace_with_export(mod, mb_args, mb_kwargs)
        pipe = Pipe._from_traced(mod, ep, multi_use_param_spec, output_loss_value_spec, split_policy,
                                 n_trace_args=len(mb_args), trace_kwarg_names=list(mb_kwargs.keys()))
        pipe.pipe_info = PipeInfo(
            graph=pipe.split_gm.graph,
            num_stages=pipe.num_stages,
            num_chunks=num_chunks,
            has_loss_and_backward=pipe.has_loss_and_backward,
            args_chunk_spec=args_spec,
            kwargs_chunk_spec=kwargs_spec,
        )
        return pipe

    @staticmethod
    def _from_traced(
        mod: nn.Module,
        exported_program,
        multi_use_param_spec: MultiUseParamSpec = MultiUseParameterConfig.REPLICATE,
        output_loss_value_spec: Any = None,
        split_policy: Optional[Callable[[fx.GraphModule], fx.GraphModule]] = None,
        n_trace_args: int = 0,
        trace_kwarg_names: Optional[List[str]] = None,
    ) -> "Pipe":
        traced = exported_program.module()
        in_spec = getattr(getattr(traced.graph, "_codegen", None), "pytree_info", None)
        in_spec = in_spec.in_spec if in_spec is not None else None
        _strip_guard_nodes(traced)
        if split_policy is not None:
            logger.info("Auto-splitting model")
            traced = split_policy(traced)
        _collapse_split_markers(traced)

        counter = [0]

        def split_callback(n: fx.Node) -> int:
            if _is_split(n):
                counter[0] += 1
            return counter[0]

        split = split_module(traced, mod, split_callback)
        split.graph.eliminate_dead_code()
        _order_stage_calls(split)
        stage_mods = [m for n, m in split.named_children() if n.startswith("submod_") and isinstance(m, fx.GraphModule)]
        num_stages = len(stage_mods)
        for sub in stage_mods:
            for node in list(sub.graph.nodes):
                if _is_split(node):
                    sub.graph.erase_node(node)
            sub.recompile()

        _sink_state_into_stages(split, mod, traced, multi_use_param_spec)

        # drop everything on the root that is not a stage module
        for name, _ in list(split.named_children()):
            if not name.startswith("submod_"):
                delattr(split, name)
        split.graph.lint()
        split.recompile()

        has_loss = False
        if output_loss_value_spec is not None or getattr(mod, "loss_spec", None) is not None:
            spec = output_loss_value_spec if output_loss_value_spec is not None else mod.loss_spec
            _insert_stage_symbolic_backward(split, spec)
            has_loss = True

        signature = None
        try:
            fwd = getattr(mod, "_pb_original_forward", None) or mod.forward
            signature = inspect.signature(fwd)
        except (TypeError, ValueError):
            signature = None
        mapping = {}
        for i in range(num_stages):
            sub = getattr(split, f"submod_{i}")
            for q, _ in sub.named_parameters(remove_duplicate=False):
                mapping[f"submod_{i}.{q}"] = q
            for q, _ in sub.named_buffers(remove_duplicate=False):
                mapping[f"submod_{i}.{q}"] = q
        return Pipe(split, num_stages, has_loss, output_loss_value_spec, signature, in_spec, n_trace_args,
                    trace_kwarg_names or [], mapping)


# ------------------------------------------------------------------------------------------------
# graph surgery helpers
# ------------------------------------------------------------------------------------------------
def _strip_guard_nodes(gm: fx.GraphModule) -> None:
    """torch.export's unlifted module carries input-guard calls; they have no users and must not become part of a
    stage."""
    for node in list(gm.graph.nodes):
        if node.op == "call_module" and str(node.target).startswith("_guards") and len(node.users) == 0:
            gm.graph.erase_node(node)
            if hasattr(gm, str(node.target)):
                delattr(gm, str(node.target))
    gm.recompile()


def _collapse_split_markers(gm: fx.GraphModule) -> None:
    """Back-to-back markers, and markers before the first or after the last computation, would create empty
    stages; keep one marker per boundary."""
    compute = [n for n in gm.graph.nodes if n.op not in ("placeholder", "get_attr", "output")]
    prev_was_split = True  # treats a leading marker as redundant
    for node in compute:
        if _is_split(node):
            if prev_was_split:
                gm.graph.erase_node(node)
                continue
            prev_was_split = True
        else:
            prev_was_split = False
    compute = [n for n in gm.graph.nodes if n.op not in ("placeholder", "get_attr", "output")]
    while compute and _is_split(compute[-1]):
        gm.graph.erase_node(compute.pop())
    gm.recompile()


def _kind_of(mod: nn.Module, qualname: str, tensor) -> Tuple[str, bool]:
    params = dict(mod.named_parameters(remove_duplicate=False))
    if qualname in params or isinstance(tensor, nn.Parameter):
        return "parameter", True
    buffers = dict(mod.named_buffers(remove_duplicate=False))
    if qualname in buffers:
        return "buffer", qualname in mod.state_dict()
    if isinstance(tensor, torch.Tensor):
        return "buffer", False
    return "constant", False


def _sink_state_into_stages(split: fx.GraphModule, mod: nn.Module, traced: fx.GraphModule,
                            multi_use_param_spec: MultiUseParamSpec) -> None:
    """Moves every tensor the root passes into a stage call to the inside of that stage, under its original name."""
    # aliases: original names that share a tensor (tied weights appear under one name in the traced graph)
    by_id: Dict[int, List[str]] = {}
    for q, t in list(mod.named_parameters(remove_duplicate=False)) + list(mod.named_buffers(remove_duplicate=False)):
        by_id.setdefault(id(t), []).append(q)

    def spec_for(qualname: str) -> MultiUseParameterConfig:
        if isinstance(multi_use_param_spec, MultiUseParameterConfig):
            return multi_use_param_spec
        if isinstance(multi_use_param_spec, dict):
            v = multi_use_param_spec.get(qualname, MultiUseParameterConfig.REPLICATE)
            if not isinstance(v, MultiUseParameterConfig):
                raise ValueError(f"Unknown multi-use config value {v} specified for {qualname}")
            return v
        raise ValueError(f"multi_use_param_spec must be MultiUseParamSpec enum or dict, got {type(multi_use_param_spec)}")

    if isinstance(multi_use_param_spec, dict):
        for q in multi_use_param_spec:
            spec_for(q)

    attr_nodes = [n for n in split.graph.nodes if n.op == "get_attr"]
    for attr in attr_nodes:
        target = str(attr.target)
        tensor = _get_by_qualname(split, target)
        users = [u for u in attr.users if u.op == "call_module"]
        users.sort(key=lambda u: int(str(u.target).split("_")[-1]))
        policy = spec_for(target) if len(users) > 1 else MultiUseParameterConfig.REPLICATE
        kind, persistent = _kind_of(mod, target, tensor)
        names = by_id.get(id(tensor), [target])
        if target not in names:
            names = [target] + names
        if policy == MultiUseParameterConfig.TRANSMIT and len(users) > 1:
            _transmit_from_first_user(split, attr, users, tensor, kind, persistent, names)
            continue
        for user in users:
            sub = getattr(split, str(user.target))
            positions = [i for i, a in enumerate(user.args) if a is attr]
            placeholders = [n for n in sub.graph.nodes if n.op == "placeholder"]
            for name in names:
                _assign_by_qualname(sub, name, tensor, kind, persistent)
            for pos in positions:
                ph = placeholders[pos]
                with sub.graph.inserting_before(ph):
                    ga = sub.graph.get_attr(target)
                    ga.meta = dict(ph.meta)
                ph.replace_all_uses_with(ga)
            for pos in sorted(positions, reverse=True):
                sub.graph.erase_node(placeholders[pos])
            user.args = tuple(a for a in user.args if a is not attr)
            sub.recompile()
        if len(attr.users) == 0:
            split.graph.erase_node(attr)
    split.recompile()


def _transmit_from_first_user(split, attr, users, tensor, kind, persistent, names) -> None:
    """TRANSMIT policy: the tensor lives in its first stage and reaches the later ones as an extra output of that
    stage (the later stages keep their placeholder)."""
    first = users[0]
    sub = getattr(split, str(first.target))
    placeholders = [n for n in sub.graph.nodes if n.op == "placeholder"]
    positions = [i for i, a in enumerate(first.args) if a is attr]
    for name in names:
        _assign_by_qualname(sub, name, tensor, kind, persistent)
    target = str(attr.target)
    ga = None
    for pos in positions:
        ph = placeholders[pos]
        with sub.graph.inserting_before(ph):
            ga = sub.graph.get_attr(target)
            ga.meta = dict(ph.meta)
        ph.replace_all_uses_with(ga)
    for pos in sorted(positions, reverse=True):
        sub.graph.erase_node(placeholders[pos])
    first.args = tuple(a for a in first.args if a is not attr)
    # make it an additional output of the first stage
    out_node = next(n for n in sub.graph.nodes if n.op == "output")
    old = out_node.args[0]
    was_tuple = isinstance(old, (tuple, list))
    new_outputs = tuple(old) + (ga,) if was_tuple else (old, ga)
    out_node.args = (new_outputs,)
    sub.recompile()
    with split.graph.inserting_after(first):
        if not was_tuple:
            # existing consumers used the stage call directly; they now take element 0
            item0 = split.graph.call_function(operator.getitem, (first, 0))
            for u in list(first.users):
                if u is not item0:
                    u.replace_input_with(first, item0)
            item0.args = (first, 0)
        with split.graph.inserting_after(first):
            transmitted = split.graph.call_function(operator.getitem, (first, len(new_outputs) - 1))
    for later in users[1:]:
        later.replace_input_with(attr, transmitted)
    if len(attr.users) == 0:
        split.graph.erase_node(attr)


# ------------------------------------------------------------------------------------------------
# loss discovery and the symbolic backward (for models that compute their loss inside forward)
# ------------------------------------------------------------------------------------------------
def _find_loss_from_output_and_spec(output_val, spec_val):
    if spec_val is False:
        return None
    if spec_val is True:
        if not isinstance(output_val, fx.Node):
            raise RuntimeError(f"Loss spec must specify a dynamic value but got {output_val}")
        return output_val
    if isinstance(spec_val, (tuple, list)):
        if not isinstance(output_val, (tuple, list)) or len(output_val) != len(spec_val):
            raise RuntimeError(f"Output value {output_val} must match the structure of loss specification {spec_val}")
        for out, spec in zip(output_val, spec_val):
            found = _find_loss_from_output_and_spec(out, spec)
            if found is not None:
                return found
        raise RuntimeError(f"Did not find loss value in specification {spec_val}")
    if isinstance(spec_val, dict):
        if not isinstance(output_val, dict) or set(output_val.keys()) != set(spec_val.keys()):
            raise RuntimeError(f"Output value {output_val} must match the structure of loss specification {spec_val}")
        for k in spec_val:
            found = _find_loss_from_output_and_spec(output_val[k], spec_val[k])
            if found is not None:
                return found
        raise RuntimeError(f"Did not find loss value in specification {spec_val}")
    raise RuntimeError(f"Unsupported type {type(spec_val)} in loss specification")


def _find_loss_output(g: fx.Graph, spec):
    output_node = next(n for n in g.nodes if n.op == "output")
    out = output_node.args[0]
    if spec is True:
        loss = out[0] if isinstance(out, (tuple, list)) and len(out) == 1 else out
        if not isinstance(loss, fx.Node):
            raise RuntimeError(f"cannot find a single loss value in output {out}")
        return loss, output_node
    if isinstance(out, (tuple, list)) and len(out) == 1 and not isinstance(spec, (tuple, list)):
        out = out[0]
    return _find_loss_from_output_and_spec(out, spec), output_node


def _order_stage_calls(split: fx.GraphModule) -> None:
    """Puts the stage calls of the split program in stage-index order, each followed by its ``getitem`` users.

    ``fx.split_module`` emits parallel branches (several stages reading one producer) in an order of its own, e.g.
    ``submod_0, submod_3, submod_2, submod_1, submod_4``.  Stage ``i`` is ``submod_i`` everywhere else (runtime
    topology, checkpoint, schedules), so the program text is made to agree.  Values only flow from a lower to a
    higher stage index, hence the index order is a valid topological order; ``lint`` checks it."""
    g = split.graph
    calls = {}
    for n in g.nodes:
        if n.op == "call_module" and str(n.target).startswith("submod_"):
            calls[int(str(n.target)[len("submod_"):])] = n
    ordered = [calls[i] for i in sorted(calls)]
    if [n for n in g.nodes if n in set(ordered)] == ordered:
        return
    cursor = None
    for n in g.nodes:
        if n.op in ("placeholder", "get_attr"):
            cursor = n
    for call in ordered:
        items = [u for u in call.users if u.op == "call_function" and u.target is operator.getitem]
        if cursor is None:
            next(iter(g.nodes)).prepend(call)
        else:
            cursor.append(call)
        cursor = call
        for u in items:
            cursor.append(u)
            cursor = u
    g.lint()
    split.recompile()


def _insert_stage_symbolic_backward(split: fx.GraphModule, loss_spec) -> None:
    """Appends one ``stage_backward`` call per stage, last stage first, to the split program so that calling the
    pipe locally also produces parameter gradients (reference _IR.py:123-232)."""
    g = split.graph
    loss_node, output_node = _find_loss_output(g, loss_spec)
    stage_calls = [n for n in g.nodes if n.op == "call_module"]
    # gradient flowing into every forward value, keyed by node
    grads: Dict[fx.Node, Optional[fx.Node]] = {}

    def producer_of(n: fx.Node) -> Optional[fx.Node]:
        if n.op == "call_module":
            return n
        if n.op == "call_function" and n.target is operator.getitem and n.args[0].op == "call_module":
            return n.args[0]
        return None

    loss_stage = producer_of(loss_node)
    if loss_stage is None:
        raise RuntimeError("the loss must be produced by a pipeline stage")
    with g.inserting_before(output_node):
        for call in reversed(stage_calls):
            outs: List[fx.Node] = []
            if any(u.op == "call_function" and u.target is operator.getitem for u in call.users):
                n_out = 1 + max(u.args[1] for u in call.users if u.op == "call_function" and u.target is operator.getitem)
                items: List[Optional[fx.Node]] = [None] * n_out
                for u in call.users:
                    if u.op == "call_function" and u.target is operator.getitem:
                        items[u.args[1]] = u
                outs = items  # type: ignore[assignment]
                multi = True
            else:
                outs = [call]
                multi = False
            if call is loss_stage:
                out_grads = None
                stage_output = loss_node
            else:
                gl = [grads.get(o) if o is not None else None for o in outs]
                if all(x is None for x in gl):
                    continue  # nothing downstream needs this stage's gradient
                stage_output = call if not multi else tuple(o if o is not None else None for o in outs)
                out_grads = gl[0] if not multi else tuple(gl)
                if multi:
                    stage_output = call
            inputs = [a for a in call.args if isinstance(a, fx.Node)]
            bw = g.call_function(
                stage_backward,
                kwargs={"stage_output": stage_output, "output_grads": out_grads, "input_values": list(inputs)},
            )
            for i, inp in enumerate(inputs):
                if producer_of(inp) is None:
                    continue
                gi = g.call_function(operator.getitem, (bw, i))
                if inp in grads and grads[inp] is not None:
                    grads[inp] = g.call_function(_null_coalesce_accumulate, (grads[inp], gi))
                else:
                    grads[inp] = gi
    split.recompile()


# ------------------------------------------------------------------------------------------------
# public entry
# ------------------------------------------------------------------------------------------------
def pipeline(
    module: nn.Module,
    num_chunks: Optional[int] = None,
    example_args: Tuple[Any, ...] = (),
    example_kwargs: Optional[Dict[str, Any]] = None,
    split_spec: Optional[Dict[str, SplitPoint]] = None,
    split_policy: Optional[Callable[[fx.GraphModule], fx.GraphModule]] = None,
    *,
    mb_args: Optional[Tuple[Any, ...]] = None,
    mb_kwargs: Optional[Dict[str, Any]] = None,
    multi_use_param_spec: MultiUseParamSpec = MultiUseParameterConfig.REPLICATE,
    output_loss_value_spec: Any = None,
) -> Pipe:
    """Splits ``module`` into pipeline stages.

    Two call styles are accepted: the reference's ``pipeline(module, num_chunks, example_args, example_kwargs, ...)``
    with FULL-batch examples (pippy/_IR.py:1341-1395), and the newer ``pipeline(module, mb_args=..., mb_kwargs=...)``
    with ONE-microbatch examples. Split points come from ``pipe_split()`` calls in the model, from ``split_spec``
    (module path -> SplitPoint) or from a ``split_policy`` (a function that annotates the traced graph).
    """
    if split_spec is not None and split_policy is not None:
        raise ValueError(
            "Cannot specify both `split_spec` and `split_policy`. Please use only one of them."
        )
    if split_spec is not None:
        annotate_split_points(module, split_spec)
    if mb_args is not None or mb_kwargs is not None:
        return Pipe.from_tracing(
            module, num_chunks, tuple(mb_args or ()), mb_kwargs, split_policy, multi_use_param_spec,
            output_loss_value_spec, already_microbatch=True,
        )
    if num_chunks is None:
        raise ValueError("pipeline() needs `num_chunks` with full-batch `example_args`, or `mb_args`/`mb_kwargs`")
    return Pipe.from_tracing(
        module, num_chunks, tuple(example_args), example_kwargs, split_policy, multi_use_param_spec,
        output_loss_value_spec,
    )


class ArgsChunkSpec:
    """Context manager: positional arguments are chunked along these dimensions while inside
    (``with ArgsChunkSpec((0, 1)): pipe = pipeline(...)``). Sets class-level state on :class:`Pipe`, as the
    reference does (pippy/_IR.py:1398-1423); the values are captured into ``PipeInfo`` at ``pipeline()`` time."""

    def __init__(self, chunk_dims: Tuple[int, ...]):
        self.args_chunk_spec = pytree.tree_map(lambda d: TensorChunkSpec(d), tuple(chunk_dims))

    def __enter__(self):
        self._prev = Pipe.args_chunk_spec
        Pipe.args_chunk_spec = self.args_chunk_spec
        return self.args_chunk_spec

    def __exit__(self, *exc):
        Pipe.args_chunk_spec = self._prev
        return False


class KwargsChunkSpec:
    """Context manager counterpart of :class:`ArgsChunkSpec` for keyword arguments: ``{name: dim}``."""

    def __init__(self, chunk_dims: Dict[str, int]):
        self.kwargs_chunk_spec = pytree.tree_map(lambda d: TensorChunkSpec(d), dict(chunk_dims))

    def __enter__(self):
        self._prev = Pipe.kwargs_chunk_spec
        Pipe.kwargs_chunk_spec = self.kwargs_chunk_spec
        return self.kwargs_chunk_spec

    def __exit__(self, *exc):
        Pipe.kwargs_chunk_spec = self._prev
        return False
