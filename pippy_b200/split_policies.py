"""Automatic split policies: functions that annotate a traced graph with ``pipe_split`` markers
(reference pippy/ModelSplit.py).  Each factory returns a ``GraphModule -> GraphModule`` callable to pass as
``pipeline(..., split_policy=...)``.

The traced graph is flat (ATen ops with ``get_attr`` nodes for parameters and buffers), so the weight of a compute
node is the number of elements of the tensors it is the FIRST to use; a tensor used again later (tied weights) is
charged once, to its first user.
"""
from __future__ import annotations

import logging
from typing import Callable, Dict, List, Tuple

import torch
import torch.fx as fx

from .ir import _is_split, aten_pipe_split_alias

logger = logging.getLogger("pippy_b200")


def _get_attr_tensor(gm: fx.GraphModule, target: str):
    obj = gm
    for atom in target.split("."):
        obj = getattr(obj, atom)
    return obj


def _analyze_node_size(gm: fx.GraphModule) -> Dict[fx.Node, int]:
    """Elements of state first used by each compute node."""
    charged = set()
    sizes: Dict[fx.Node, int] = {}
    for node in gm.graph.nodes:
        if node.op in ("placeholder", "get_attr", "output"):
            continue
        total = 0
        for inp in node.all_input_nodes:
            if inp.op == "get_attr" and inp not in charged:
                t = _get_attr_tensor(gm, str(inp.target))
                if isinstance(t, torch.Tensor):
                    total += t.numel()
                charged.add(inp)
        sizes[node] = total
    return sizes


def _total_state_size(gm: fx.GraphModule) -> int:
    seen = set()
    total = 0
    for node in gm.graph.nodes:
        if node.op == "get_attr" and node.target not in seen:
            seen.add(node.target)
            t = _get_attr_tensor(gm, str(node.target))
            if isinstance(t, torch.Tensor):
                total += t.numel()
    return total


def _split_on_size_threshold_with_max_stages(gm: fx.GraphModule, threshold: int, max_stages: int = -1) -> Tuple[fx.GraphModule, int]:
    sizes = _analyze_node_size(gm)
    accumulated = 0
    stages = 1
    compute = [n for n in gm.graph.nodes if n.op not in ("placeholder", "get_attr", "output")]
    for i, node in enumerate(compute):
        if _is_split(node):
            continue
        w = sizes.get(node, 0)
        # open a new stage before a node that would overflow a non-empty bucket
        if accumulated > 0 and accumulated + w > threshold and (max_stages < 0 or stages < max_stages):
            with gm.graph.inserting_before(node):
                gm.graph.call_function(aten_pipe_split_alias, (), {})
            stages += 1
            accumulated = 0
        accumulated += w
    gm.graph.lint()
    gm.recompile()
    return gm, stages


def split_on_size_threshold(threshold: int) -> Callable[[fx.GraphModule], fx.GraphModule]:
    """Greedy: start a new stage whenever the current one would exceed ``threshold`` elements of state."""

    def policy(gm: fx.GraphModule) -> fx.GraphModule:
        gm, n = _split_on_size_threshold_with_max_stages(gm, threshold)
        logger.info("split_on_size_threshold(%d) produced %d stages", threshold, n)
        return gm

    return policy


def split_into_equal_size(nstages: int = 1) -> Callable[[fx.GraphModule], fx.GraphModule]:
    """Splits into exactly ``nstages`` stages of roughly equal parameter+buffer size."""

    def policy(gm: fx.GraphModule) -> fx.GraphModule:
        total = _total_state_size(gm)
        threshold = max(total // nstages, 1)
        gm, n = _split_on_size_threshold_with_max_stages(gm, threshold, nstages)
        if n != nstages:
            # too few heavy nodes to reach the count by size alone: cut the remaining compute evenly
            compute = [x for x in gm.graph.nodes if x.op not in ("placeholder", "get_attr", "output") and not _is_split(x)]
            existing = [x for x in gm.graph.nodes if _is_split(x)]
            missing = nstages - n
            if len(compute) > missing + len(existing):
                step = len(compute) // (missing + 1)
                for k in range(1, missing + 1):
                    node = compute[min(k * step, len(compute) - 1)]
                    prev = node.prev
                    if _is_split(node) or _is_split(prev):
                        continue
                    with gm.graph.inserting_before(node):
                        gm.graph.call_function(aten_pipe_split_alias, (), {})
                    n += 1
                gm.graph.lint()
                gm.recompile()
        assert n == nstages, f"split_into_equal_size produced {n} stages instead of {nstages}"
        return gm

    return policy


def split_by_graph(nstages: int) -> Callable[[fx.GraphModule], fx.GraphModule]:
    """Balanced split that also minimises inter-stage traffic, solved as a mixed-integer program."""

    def policy(gm: fx.GraphModule) -> fx.GraphModule:
        from .graphsplit import split_by_graph_with_num_stages

        return split_by_graph_with_num_stages(gm, nstages)

    return policy
