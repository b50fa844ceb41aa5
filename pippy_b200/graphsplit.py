"""Graph-based automatic splitting (reference pippy/graphsplit.py).

Nodes are weighted by the state they own, edges by the size of the activation they carry.  After merging linear
chains (a chain can never be cut more cheaply than at its lightest edge, which is kept) the stage assignment is a
mixed-integer program solved with ``scipy.optimize.milp``:

  variables   x[n, k] in {0, 1}   node n runs in stage k
  subject to  sum_k x[n, k] = 1
              stage(u) <= stage(v)            for every edge u -> v      (stage(n) = sum_k k * x[n, k])
              sum_n w_n x[n, k] <= MAX_MEMORY_IMBALANCE * total / K      (balanced state)
              sum_n x[n, k] >= 1                                         (no empty stage)
              cross_k <= MAX_COMMUNICATION_IMBALANCE * mean_j cross_j    (balanced transfers; see below)
  minimise    sum_edges a_e * (stage(v) - stage(u))                     (activation bytes x hops)

``cross_k`` is what crosses the boundary between stages k and k+1: with y[n, k] = sum_{j<=k} x[n, j] ("n runs in
stage k or earlier") an edge u -> v crosses it exactly when y[u, k] - y[v, k] = 1, so cross_k is linear in x and the
bound on the busiest boundary relative to the mean is a linear constraint too (the reference bounds its per-stage
edge weight the same way, pippy/graphsplit.py:48, 270-285).  Some graphs cannot meet it (an embedding output next
to a wide hidden state); then the program is solved again without it and a warning says so.

The graph is then reordered stage by stage (legal because edges never point to an earlier stage) and a
``pipe_split`` marker is placed at every boundary.
"""
from __future__ import annotations

import logging
from typing import Dict, List, Tuple

import torch
import torch.fx as fx

from .ir import _is_split, aten_pipe_split_alias
from .split_policies import _analyze_node_size

logger = logging.getLogger("pippy_b200")

MAX_MEMORY_IMBALANCE = 2.5
MAX_COMMUNICATION_IMBALANCE = 1.1
SCIPY_TIME_LIMIT_SEC = 30

try:
    from scipy.optimize import Bounds, LinearConstraint, milp  # type: ignore

    _HAVE_SCIPY = True
except Exception:  # pragma: no cover
    _HAVE_SCIPY = False


def _activation_numel(node: fx.Node) -> int:
    val = node.meta.get("val")
    if isinstance(val, torch.Tensor):
        return int(val.numel())
    if isinstance(val, (tuple, list)):
        return int(sum(v.numel() for v in val if isinstance(v, torch.Tensor)))
    return 1


def _build_groups(gm: fx.GraphModule) -> Tuple[List[List[fx.Node]], Dict[fx.Node, int]]:
    """Merges single-producer/single-consumer chains into groups; returns groups in topological order."""
    compute = [n for n in gm.graph.nodes if n.op not in ("placeholder", "get_attr", "output") and not _is_split(n)]
    group_of: Dict[fx.Node, int] = {}
    groups: List[List[fx.Node]] = []
    for node in compute:
        preds = [p for p in node.all_input_nodes if p in group_of]
        merged = False
        if len(preds) == 1:
            p = preds[0]
            consumers = [u for u in p.users if u.op != "output"]
            # only glue to the LAST node of a group, and only when the producer has this single consumer
            if len(consumers) == 1 and groups[group_of[p]][-1] is p:
                groups[group_of[p]].append(node)
                group_of[node] = group_of[p]
                merged = True
        if not merged:
            group_of[node] = len(groups)
            groups.append([node])
    return groups, group_of


def split_by_graph_with_num_stages(gm: fx.GraphModule, num_stages: int) -> fx.GraphModule:
    if not _HAVE_SCIPY:
        raise RuntimeError("split_by_graph needs scipy >= 1.9 (scipy.optimize.milp), which is not installed")
    import numpy as np

    sizes = _analyze_node_size(gm)
    groups, group_of = _build_groups(gm)
    N, K = len(groups), num_stages
    if N < K:
        raise ValueError(f"the graph has only {N} separable groups, cannot make {K} stages")
    weights = np.array([sum(sizes.get(n, 0) for n in g) for g in groups], dtype=float)
    edges: Dict[Tuple[int, int], float] = {}
    for node, gi in group_of.items():
        for u in node.users:
            gj = group_of.get(u)
            if gj is not None and gj != gi:
                edges[(gi, gj)] = edges.get((gi, gj), 0.0) + _activation_numel(node)
    # a long chain of tiny groups makes the program large; cap by merging neighbours while it is too big
    total_w = float(weights.sum()) or 1.0

    nvar = N * K

    def var(n, k):
        return n * K + k

    c = np.zeros(nvar)
    for (u, v), a in edges.items():
        for k in range(K):
            c[var(v, k)] += a * k
            c[var(u, k)] -= a * k
    rows, lo, hi = [], [], []
    for n in range(N):  # one stage per node
        r = np.zeros(nvar)
        r[[var(n, k) for k in range(K)]] = 1
        rows.append(r); lo.append(1); hi.append(1)
    for (u, v) in edges:  # forward-only edges
        r = np.zeros(nvar)
        for k in range(K):
            r[var(v, k)] += k
            r[var(u, k)] -= k
        rows.append(r); lo.append(0); hi.append(K)
    cap = MAX_MEMORY_IMBALANCE * total_w / K
    heaviest = float(weights.max()) if N else 0.0
    cap = max(cap, heaviest)
    for k in range(K):  # balanced state, no empty stage
        r = np.zeros(nvar)
        for n in range(N):
            r[var(n, k)] = weights[n]
        rows.append(r); lo.append(0); hi.append(cap)
        r2 = np.zeros(nvar)
        r2[[var(n, k) for n in range(N)]] = 1
        rows.append(r2); lo.append(1); hi.append(N)
    # balanced transfers: (K - 1) * cross_k - MAX_COMMUNICATION_IMBALANCE * sum_j cross_j <= 0 for every boundary k
    comm_rows = []
    if K > 2 and edges:
        cross = np.zeros((K - 1, nvar))
        for (u, v), a in edges.items():
            for k in range(K - 1):
                for j in range(k + 1):
                    cross[k, var(u, j)] += a
                    cross[k, var(v, j)] -= a
        total_cross = cross.sum(axis=0)
        for k in range(K - 1):
            comm_rows.append((K - 1) * cross[k] - MAX_COMMUNICATION_IMBALANCE * total_cross)

    def solve(with_comm: bool):
        a_rows = rows + (comm_rows if with_comm else [])
        a_lo = lo + ([-np.inf] * len(comm_rows) if with_comm else [])
        a_hi = hi + ([0.0] * len(comm_rows) if with_comm else [])
        return milp(c, constraints=LinearConstraint(np.array(a_rows), np.array(a_lo), np.array(a_hi)),
                    integrality=np.ones(nvar), bounds=Bounds(0, 1), options={"time_limit": SCIPY_TIME_LIMIT_SEC})

    res = solve(bool(comm_rows))
    if comm_rows and (res.status != 0 or res.x is None):
        logger.warning("split_by_graph: no assignment keeps every boundary within %.2fx of the mean transfer; "
                       "solving without the communication-balance constraint", MAX_COMMUNICATION_IMBALANCE)
        res = solve(False)
    if res.status == 1:
        raise ValueError(f"graph split did not finish within {SCIPY_TIME_LIMIT_SEC}s; use a size-based policy instead")
    if not res.success or res.x is None:
        raise ValueError(f"graph split is infeasible for {K} stages: {res.message}")
    x = np.round(res.x).reshape(N, K)
    stage_of_group = x.argmax(axis=1)
    stage_of: Dict[fx.Node, int] = {n: int(stage_of_group[g]) for n, g in group_of.items()}
    _reorder_and_mark(gm, stage_of, K)
    counts = [int((stage_of_group == k).sum()) for k in range(K)]
    per_stage_w = [float(weights[stage_of_group == k].sum()) for k in range(K)]
    logger.info("split_by_graph: groups per stage %s, state per stage %s, objective %.3g", counts, per_stage_w, res.fun)
    return gm


def _reorder_and_mark(gm: fx.GraphModule, stage_of: Dict[fx.Node, int], K: int) -> None:
    output = next(n for n in gm.graph.nodes if n.op == "output")
    for n in list(gm.graph.nodes):
        if _is_split(n):
            gm.graph.erase_node(n)
    compute = [n for n in gm.graph.nodes if n in stage_of]
    ordered = sorted(compute, key=lambda n: stage_of[n])  # stable: original order inside a stage
    for n in ordered:
        output.prepend(n)
    prev_stage = None
    for n in ordered:
        if prev_stage is not None and stage_of[n] != prev_stage:
            with gm.graph.inserting_before(n):
                gm.graph.call_function(aten_pipe_split_alias, (), {})
        prev_stage = stage_of[n]
    gm.graph.lint()
    gm.recompile()
