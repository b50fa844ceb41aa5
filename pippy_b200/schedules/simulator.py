"""Replays a schedule against a cost model: makespan, per-rank bubble fraction, peak in-flight microbatches.

Used by the tests to pin schedule properties (for example: zero-bubble has a smaller bubble than 1F1B at equal
cost) and by users to choose a schedule before spending GPU time.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

from .actions import Action, Op, Schedule, ScheduleDeadlock, _sources, linear_topology


@dataclass
class SimResult:
    makespan: float
    busy: Dict[int, float]
    bubble: Dict[int, float]            # 1 - busy / makespan, per rank
    peak_in_flight: Dict[int, int]      # forwards whose backward (B or I) has not run yet
    peak_pending_w: Dict[int, int]
    timeline: Dict[int, List[Tuple[float, float, Action]]] = field(default_factory=dict)

    @property
    def max_bubble(self) -> float:
        return max(self.bubble.values())

    @property
    def mean_bubble(self) -> float:
        return sum(self.bubble.values()) / len(self.bubble)


def simulate(
    schedule: Schedule,
    stage_to_rank: Callable[[int], int],
    num_stages: int,
    cost: Optional[Dict[Op, float]] = None,
    comm_latency: float = 0.0,
    dests: Optional[Dict[int, List[int]]] = None,
) -> SimResult:
    """Event-driven replay. Communication actions are free; a remote dependency becomes visible
    ``comm_latency`` after its producer finishes."""
    cost = cost or {Op.F: 1.0, Op.B: 2.0, Op.I: 1.0, Op.W: 1.0}
    dests = dests if dests is not None else linear_topology(num_stages)
    srcs = _sources(dests)
    ranks = sorted(schedule)
    compute = {r: [a for a in schedule[r] if a.op.is_compute] for r in ranks}
    ptr = {r: 0 for r in ranks}
    clock = {r: 0.0 for r in ranks}
    busy = {r: 0.0 for r in ranks}
    finish: Dict[tuple, float] = {}
    in_flight = {r: 0 for r in ranks}
    pend_w = {r: 0 for r in ranks}
    peak = {r: 0 for r in ranks}
    peak_w = {r: 0 for r in ranks}
    timeline: Dict[int, List[Tuple[float, float, Action]]] = {r: [] for r in ranks}

    def dep_time(a: Action, r: int) -> Optional[float]:
        times = [0.0]

        def need(key, producer_stage):
            t = finish.get(key)
            if t is None:
                return False
            times.append(t + (comm_latency if stage_to_rank(producer_stage) != r else 0.0))
            return True

        if a.op == Op.F:
            for s in srcs.get(a.stage, []):
                if not need((s, "F", a.mb), s):
                    return None
        elif a.op in (Op.B, Op.I):
            if not need((a.stage, "F", a.mb), a.stage):
                return None
            for d in dests.get(a.stage, []):
                if not need((d, "BI", a.mb), d):
                    return None
        elif a.op == Op.W:
            if not need((a.stage, "BI", a.mb), a.stage):
                return None
        return max(times)

    progressed = True
    while progressed:
        progressed = False
        for r in ranks:
            while ptr[r] < len(compute[r]):
                a = compute[r][ptr[r]]
                t_dep = dep_time(a, r)
                if t_dep is None:
                    break
                start = max(clock[r], t_dep)
                end = start + cost[a.op]
                clock[r] = end
                busy[r] += cost[a.op]
                timeline[r].append((start, end, a))
                if a.op == Op.F:
                    finish[(a.stage, "F", a.mb)] = end
                    in_flight[r] += 1
                    peak[r] = max(peak[r], in_flight[r])
                elif a.op in (Op.B, Op.I):
                    finish[(a.stage, "BI", a.mb)] = end
                    in_flight[r] -= 1
                    if a.op == Op.I:
                        pend_w[r] += 1
                        peak_w[r] = max(peak_w[r], pend_w[r])
                else:
                    pend_w[r] -= 1
                ptr[r] += 1
                progressed = True
    if any(ptr[r] < len(compute[r]) for r in ranks):
        stuck = {r: compute[r][ptr[r]] for r in ranks if ptr[r] < len(compute[r])}
        raise ScheduleDeadlock(f"schedule deadlocks in simulation; blocked at {stuck}")
    makespan = max(clock.values()) if clock else 0.0
    bubble = {r: (1.0 - busy[r] / makespan) if makespan > 0 else 0.0 for r in ranks}
    return SimResult(makespan, busy, bubble, peak, peak_w, timeline)


def ideal_bubble(P: int, n_mb: int, v: int = 1) -> float:
    """Analytic bubble fraction of GPipe/1F1B (v=1) and interleaved 1F1B: (P-1)/(v*m + P-1)."""
    return (P - 1) / (v * n_mb + P - 1)
