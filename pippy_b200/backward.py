"""Per-stage backward passes.

* :func:`stage_backward` – full backward of one microbatch through one stage (reference pippy/_backward.py:9-102).
* :func:`stage_backward_input` / :func:`stage_backward_weight` – the split used by zero-bubble schedules: the
  input-gradient half runs on the critical path, the weight-gradient half is deferred
  (upstream torch/distributed/pipelining/_backward.py:143-279 describes the same contract).  Two mechanisms are
  combined: layers of this package (``ops.linear``) park their weight-gradient GEMMs in a
  :class:`DeferredWeightGrads` queue while the input half runs, and anything else falls back to an
  autograd-graph walk that stops at the parameters' producers.
"""
from __future__ import annotations

import collections
import threading
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch

from ._debug import map_debug_info


def _flatten_outputs_and_grads(stage_output, output_grads) -> Tuple[List[torch.Tensor], List[Optional[torch.Tensor]]]:
    outs: List[torch.Tensor] = []
    grads: List[Optional[torch.Tensor]] = []

    def visit(out, grad):
        if isinstance(out, torch.Tensor):
            if not out.requires_grad and out.grad_fn is None:
                return
            if grad is not None and not isinstance(grad, torch.Tensor):
                raise TypeError(f"gradient for a tensor output must be a tensor or None, got {type(grad)}")
            outs.append(out)
            grads.append(grad)
        elif isinstance(out, (tuple, list)):
            if grad is None:
                return
            if not isinstance(grad, (tuple, list)) or len(grad) != len(out):
                raise TypeError(f"output is a sequence of {len(out)} but its gradients are {type(grad)}")
            for o, g in zip(out, grad):
                visit(o, g)
        elif isinstance(out, dict):
            if grad is None:
                return
            if not isinstance(grad, dict) or set(grad.keys()) != set(out.keys()):
                raise TypeError("output is a dict but its gradients do not have the same keys")
            for k in out.keys():
                visit(out[k], grad[k])
        # anything else carries no gradient

    visit(stage_output, output_grads)
    return outs, grads


def stage_backward(
    stage_output,
    output_grads,
    input_values: Sequence[Any],
    outputs_with_grads_idxs: Optional[List[int]] = None,
) -> List[Optional[torch.Tensor]]:
    """Backpropagates ``output_grads`` through the autograd graph of ``stage_output``.

    Parameter gradients accumulate into ``.grad``; the return value lists the gradient of every entry of
    ``input_values`` (``None`` for non-tensors and tensors without gradient).  For the last stage pass the loss
    as ``stage_output`` and ``None`` as ``output_grads``.
    """
    if outputs_with_grads_idxs is not None:
        stage_output = [stage_output[i] for i in outputs_with_grads_idxs]
        output_grads = [output_grads[i] for i in outputs_with_grads_idxs]
    try:
        if output_grads is None and isinstance(stage_output, torch.Tensor):
            outs, grads = [stage_output], [None]
        elif output_grads is None and isinstance(stage_output, (tuple, list)):
            outs = [o for o in stage_output if isinstance(o, torch.Tensor) and (o.requires_grad or o.grad_fn)]
            grads = [None] * len(outs)
        else:
            outs, grads = _flatten_outputs_and_grads(stage_output, output_grads)
        live = [(o, g) for o, g in zip(outs, grads) if not (g is None and o.numel() != 1)]
        if live:
            torch.autograd.backward([o for o, _ in live], grad_tensors=[g for _, g in live])
        result: List[Optional[torch.Tensor]] = []
        for v in input_values:
            result.append(v.grad if isinstance(v, torch.Tensor) else None)
        return result
    except Exception as e:
        raise RuntimeError(
            f"""
        Failed to run stage backward:
        Stage output: {map_debug_info(stage_output)}
        Output gradient: {map_debug_info(output_grads)}
        Input: {map_debug_info(list(input_values))}
        """
        ) from e


def _null_coalesce_accumulate(lhs, rhs):
    """``lhs + rhs`` where either side may be ``None`` (reference _backward.py:107-117)."""
    if lhs is None:
        return rhs
    if rhs is None:
        return lhs
    return torch.add(lhs, rhs)


# --------------------------------------------------------------------------------------------
# Deferred weight gradients (the fast path for this package's own layers)
# --------------------------------------------------------------------------------------------
class DeferredWeightGrads:
    """FIFO of weight-gradient closures recorded while an input-gradient pass runs.

    A layer's autograd backward asks :func:`current_deferral` for the active queue; when there is one it
    computes only the input gradient and calls :meth:`defer` with a closure that, when run later, accumulates the
    weight gradient.
    """

    def __init__(self) -> None:
        self._items: List[Callable[[], None]] = []

    def defer(self, fn: Callable[[], None]) -> None:
        self._items.append(fn)

    def __len__(self) -> int:
        return len(self._items)

    def run(self) -> None:
        items, self._items = self._items, []
        for fn in items:
            fn()


# Process-wide on purpose: autograd runs the backward of CUDA ops on its own device thread, so a thread-local set by
# the caller would be invisible there.  The schedule runs one action at a time, so a single slot is enough.
class _DeferralState:
    queue: Optional["DeferredWeightGrads"] = None


_tls = _DeferralState


def current_deferral() -> Optional[DeferredWeightGrads]:
    return _tls.queue


class defer_weight_grads:
    """Context manager: weight-gradient work of this package's layers goes to ``queue`` instead of running."""

    def __init__(self, queue: Optional[DeferredWeightGrads]):
        self.queue = queue

    def __enter__(self):
        self.prev = _tls.queue
        _tls.queue = self.queue
        return self.queue

    def __exit__(self, *exc):
        _tls.queue = self.prev
        return False


# --------------------------------------------------------------------------------------------
# Generic split for arbitrary modules: walk the autograd graph
# --------------------------------------------------------------------------------------------
def _grad_fn_of(t: torch.Tensor):
    if t.grad_fn is not None:
        return t.grad_fn
    if t.requires_grad:
        return torch.autograd.graph.get_gradient_edge(t).node  # AccumulateGrad of a leaf
    return None


def _reachable_from(roots: Iterable[Any]) -> set:
    seen = set()
    stack = [r for r in roots if r is not None]
    while stack:
        node = stack.pop()
        if node in seen:
            continue
        seen.add(node)
        for nxt, _ in node.next_functions:
            if nxt is not None and nxt not in seen:
                stack.append(nxt)
    return seen


class _WeightGradPlan:
    """What :func:`stage_backward_input` leaves behind for :func:`stage_backward_weight`."""

    def __init__(self) -> None:
        self.deferred: Optional[DeferredWeightGrads] = None
        # (gradient edges of a split node, the gradients captured there, parameters below its off-path children)
        self.boundaries: List[Tuple[Tuple[Any, ...], Tuple[torch.Tensor, ...], List[torch.nn.Parameter]]] = []
        self.full_backward: Optional[Tuple[List[torch.Tensor], List[Optional[torch.Tensor]]]] = None


def stage_backward_input(
    stage_outputs_or_loss: Sequence[torch.Tensor],
    output_grads: Optional[Sequence[Optional[torch.Tensor]]],
    input_values: Sequence[torch.Tensor],
    weights: Iterator[torch.nn.Parameter],
) -> Tuple[List[Optional[torch.Tensor]], _WeightGradPlan]:
    """Computes only the gradients of ``input_values``; parameter gradients are postponed.

    Returns ``(input_grads, plan)``; hand ``plan`` to :func:`stage_backward_weight` to finish. When no input
    requires a gradient (the first stage) nothing is computed now and the plan holds a full backward.
    """
    outs = [o for o in stage_outputs_or_loss if isinstance(o, torch.Tensor) and (o.requires_grad or o.grad_fn)]
    if output_grads is None:
        grads: List[Optional[torch.Tensor]] = [None] * len(outs)
    else:
        pairs = [
            (o, g)
            for o, g in zip(stage_outputs_or_loss, output_grads)
            if isinstance(o, torch.Tensor) and (o.requires_grad or o.grad_fn) and g is not None
        ]
        outs = [o for o, _ in pairs]
        grads = [g for _, g in pairs]
    grads = [g if g is not None else torch.ones_like(o) for o, g in zip(outs, grads)]

    plan = _WeightGradPlan()
    diff_inputs = [v for v in input_values if isinstance(v, torch.Tensor) and v.requires_grad]
    # parameters whose owning op writes their gradient itself (ops.functional) never go through the graph walk
    weights = [w for w in weights if w.requires_grad and not getattr(w, "_pb_direct_grad", False)]
    if not diff_inputs:
        # First stage: nobody waits for an input gradient, but the chain of activation gradients still has to run
        # to reach the early layers' parameters.  Run it now with deferral on: layers of this package queue their
        # weight-gradient GEMMs for the W action (so I and W cost about what they cost on every other stage, which
        # keeps the schedule balanced); parameters of other ops simply get their gradient during this pass.
        if outs:
            queue = DeferredWeightGrads()
            plan.deferred = queue
            with defer_weight_grads(queue):
                torch.autograd.backward(outs, grad_tensors=grads)
        return [None] * len(input_values), plan
    if not outs:
        return [None] * len(input_values), plan

    # Nodes on a path output -> input.  A node *off* that path whose parent is *on* it is a boundary: its
    # gradient is what the weight half needs.  Hooks capture those gradients during the input pass.
    input_nodes = {_grad_fn_of(v) for v in diff_inputs}
    weight_nodes = {}
    for w in weights:
        node = _grad_fn_of(w)
        if node is not None:
            weight_nodes.setdefault(node, []).append(w)

    # reverse reachability: which nodes can reach an input leaf
    out_roots = [o.grad_fn for o in outs if o.grad_fn is not None]
    order: List[Any] = []
    seen = set()
    stack = [(r, False) for r in out_roots]
    while stack:
        node, done = stack.pop()
        if done:
            order.append(node)
            continue
        if node in seen:
            continue
        seen.add(node)
        stack.append((node, True))
        for nxt, _ in node.next_functions:
            if nxt is not None and nxt not in seen:
                stack.append((nxt, False))
    reaches_input = set()
    for node in order:  # children before parents
        if node in input_nodes or any(n is not None and n in reaches_input for n, _ in node.next_functions):
            reaches_input.add(node)

    # Split points: nodes ON the input path with at least one child OFF it that leads to parameters.  The gradient
    # arriving at such a node is captured during the input pass; the weight pass restarts autograd from the node
    # with that gradient and asks only for the parameters hanging below its off-path children.
    below_cache: Dict[Any, List[torch.nn.Parameter]] = {}

    def weights_below(node) -> List[torch.nn.Parameter]:
        hit = below_cache.get(node)
        if hit is not None:
            return hit
        found: List[torch.nn.Parameter] = []
        for n in _reachable_from([node]):
            found.extend(weight_nodes.get(n, ()))
        below_cache[node] = found
        return found

    split_nodes: List[Tuple[Any, List[torch.nn.Parameter]]] = []
    claimed: Dict[int, int] = {}
    conflict = False
    for node in order:
        if node not in reaches_input:
            continue
        off_params: List[torch.nn.Parameter] = []
        for child, _slot in node.next_functions:
            if child is None or child in reaches_input:
                continue
            off_params.extend(weights_below(child))
        if not off_params:
            continue
        uniq = list({id(p): p for p in off_params}.values())
        for p_ in uniq:
            claimed[id(p_)] = claimed.get(id(p_), 0) + 1
            if claimed[id(p_)] > 1:
                conflict = True  # a parameter reachable from two split points would be counted twice
        split_nodes.append((node, uniq))
    # outputs whose whole history is off the input path contribute only to parameters
    weight_only_outputs = []
    for o, g in zip(outs, grads):
        node = o.grad_fn
        if node is not None and node not in reaches_input and weights_below(node):
            weight_only_outputs.append((o, g))
            for p_ in weights_below(node):
                claimed[id(p_)] = claimed.get(id(p_), 0) + 1
                if claimed[id(p_)] > 1:
                    conflict = True

    if conflict:
        # exact split is not possible with this graph shape: run the whole backward now, nothing is deferred
        torch.autograd.backward(outs, grad_tensors=grads)
        return [v.grad if isinstance(v, torch.Tensor) else None for v in input_values], plan

    queue = DeferredWeightGrads()
    plan.deferred = queue
    captured: Dict[Any, Tuple[Optional[torch.Tensor], ...]] = {}
    handles = []

    def make_hook(node):
        def hook(grad_outputs):
            prev = captured.get(node)
            if prev is None:
                captured[node] = tuple(grad_outputs)
            else:
                captured[node] = tuple(_null_coalesce_accumulate(a, b) for a, b in zip(prev, grad_outputs))
            return None

        return hook

    for node, _params in split_nodes:
        handles.append(node.register_prehook(make_hook(node)))
    # The graph has to survive only if the weight half will re-enter it; when every parameter gradient is deferred
    # through the queue (the package's own layers) the saved activations are released as the input pass consumes them.
    keep_graph = bool(split_nodes) or bool(weight_only_outputs)
    try:
        with defer_weight_grads(queue):
            in_grads = torch.autograd.grad(outs, diff_inputs, grad_outputs=grads, retain_graph=keep_graph,
                                           allow_unused=True)
    finally:
        for h in handles:
            h.remove()

    for node, params in split_nodes:
        got = captured.get(node)
        if got is None:
            continue
        edges = []
        edge_grads = []
        for slot, g in enumerate(got):
            if g is not None:
                edges.append(torch.autograd.graph.GradientEdge(node, slot))
                edge_grads.append(g)
        if edges:
            plan.boundaries.append((tuple(edges), tuple(edge_grads), params))
    for o, g in weight_only_outputs:
        edge = torch.autograd.graph.get_gradient_edge(o)
        plan.boundaries.append(((edge,), (g,), weights_below(o.grad_fn)))

    result: List[Optional[torch.Tensor]] = []
    it = iter(in_grads)
    for v in input_values:
        if isinstance(v, torch.Tensor) and v.requires_grad:
            g = next(it)
            result.append(g)
        else:
            result.append(None)
    return result, plan


def stage_backward_weight(weights: Iterator[torch.nn.Parameter], plan: _WeightGradPlan, retain_graph: bool = False) -> None:
    """Finishes what :func:`stage_backward_input` postponed: accumulates parameter gradients into ``.grad``."""
    if plan.full_backward is not None:
        outs, grads = plan.full_backward
        if outs:
            torch.autograd.backward(outs, grad_tensors=grads, retain_graph=retain_graph)
        plan.full_backward = None
        return
    if plan.deferred is not None:
        plan.deferred.run()
    if plan.boundaries:
        # group by parameter set so each autograd.grad call touches its own subgraph once
        for edges, grads, params in plan.boundaries:
            params = [p for p in params if p.requires_grad]
            if not params:
                continue
            with defer_weight_grads(None):
                dws = torch.autograd.grad(edges, params, grad_outputs=grads, retain_graph=True, allow_unused=True)
            for p, dw in zip(params, dws):
                if dw is None:
                    continue
                if p.grad is None:
                    p.grad = dw.detach()
                else:
                    p.grad = p.grad + dw
        plan.boundaries = []
