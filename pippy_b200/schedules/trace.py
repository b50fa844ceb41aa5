"""Chrome-trace (chrome://tracing, Perfetto) views of a schedule: the plan replayed on a cost model, and the
measured timeline of a step.

The reference has no such view of its own; users wrap ``schedule.step`` in ``torch.profiler`` and export a trace
per rank (reference examples/profiling/mlp_profiling.py:87-101), which still works here because every compute
action runs inside a ``record_function`` range.  These dumps are smaller and line the ranks up on one time axis.
"""
from __future__ import annotations

import json
from typing import Any, Dict, Iterable, List, Optional, Tuple

from .actions import Op, Schedule
from .simulator import SimResult

_COLOURS = {"F": "thread_state_running", "B": "thread_state_iowait", "I": "thread_state_iowait",
            "W": "thread_state_runnable"}


def _event(name: str, op: str, rank: int, start_us: float, dur_us: float) -> Dict[str, Any]:
    ev = {"name": name, "cat": op, "ph": "X", "pid": 0, "tid": rank, "ts": start_us, "dur": dur_us}
    if op in _COLOURS:
        ev["cname"] = _COLOURS[op]
    return ev


def simulated_trace(result: SimResult, unit_us: float = 1000.0) -> List[Dict[str, Any]]:
    """Events of a simulated schedule (``simulate(...)``), one row per rank; one cost unit = ``unit_us``."""
    events = []
    for rank, items in sorted(result.timeline.items()):
        for start, end, action in items:
            events.append(_event(str(action), action.op.value, rank, start * unit_us, (end - start) * unit_us))
    return events


def measured_trace(stats: Dict[str, Any], rank: int) -> List[Dict[str, Any]]:
    """Events of one measured step (``schedule.last_step_stats`` with ``record_timing=True``) of one rank."""
    events = []
    for name, t0, t1 in stats["timeline"]:
        op = name.split("(")[0].strip() if "(" in name else "".join(c for c in name if c.isalpha())
        events.append(_event(name, op, rank, t0 * 1e6, (t1 - t0) * 1e6))
    return events


def write_chrome_trace(path: str, events: Iterable[Dict[str, Any]], rank_names: Optional[Dict[int, str]] = None) -> None:
    events = list(events)
    meta = [{"name": "thread_name", "ph": "M", "pid": 0, "tid": r, "args": {"name": n}}
            for r, n in (rank_names or {}).items()]
    with open(path, "w") as f:
        json.dump({"traceEvents": meta + events, "displayTimeUnit": "ms"}, f)


def gather_measured_trace(schedule, path: str, group=None) -> None:
    """Collects every rank's measured timeline of the last step on rank 0 of ``group`` and writes one trace file.
    The ranks' clocks are their own step starts, which the step's first receive aligns to within a message latency."""
    import torch.distributed as dist

    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    mine = measured_trace(schedule.last_step_stats, rank)
    if world > 1:
        gathered: List[Any] = [None] * world
        dist.all_gather_object(gathered, mine, group=group)
    else:
        gathered = [mine]
    if rank == 0:
        write_chrome_trace(path, [e for part in gathered for e in part], {r: f"rank {r}" for r in range(world)})
