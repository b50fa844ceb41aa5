"""Schedule-as-data: the vocabulary every pipeline schedule is written in.

A schedule is, per pipeline rank, a flat list of :class:`Action` records.  Pure functions
(``generators.py``) produce the compute actions, :func:`add_send_recv` threads the communication actions
through them, ``simulator.py`` replays a schedule against a cost model (bubble fraction, peak in-flight
microbatches) and ``runtime.py`` executes it on a stage.  The reference drives its schedules with imperative
loops (pippy/PipelineSchedule.py:279-778); upstream's later runtime uses a similar action list
(torch/distributed/pipelining/schedules.py:45-180).
"""
from __future__ import annotations

import csv
import enum
import re
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence


class Op(enum.Enum):
    F = "F"            # forward of one microbatch through one stage
    B = "B"            # full backward (input + weight gradients)
    I = "I"            # input-gradient half of the backward  # noqa: E741
    W = "W"            # weight-gradient half of the backward
    SEND_F = "SEND_F"  # send stage outputs of a microbatch downstream
    RECV_F = "RECV_F"  # post the receive of stage inputs
    SEND_B = "SEND_B"  # send input gradients upstream
    RECV_B = "RECV_B"  # post the receive of output gradients
    REDUCE_GRAD = "REDUCE_GRAD"  # data-parallel gradient reduction of a stage (after its last backward)

    @property
    def is_compute(self) -> bool:
        return self in (Op.F, Op.B, Op.I, Op.W)

    @property
    def is_comm(self) -> bool:
        return self in (Op.SEND_F, Op.RECV_F, Op.SEND_B, Op.RECV_B)


@dataclass(frozen=True)
class Action:
    """One step of one rank's schedule. ``peer`` is the stage on the other end of a RECV (None = every source)."""

    stage: int
    op: Op
    mb: Optional[int] = None
    peer: Optional[int] = None

    def __str__(self) -> str:
        s = f"{self.stage}{self.op.value}"
        if self.mb is not None:
            s += str(self.mb)
        if self.peer is not None:
            s += f"@{self.peer}"
        return s

    __repr__ = __str__

    _PATTERN = re.compile(r"^(\d+)(SEND_F|RECV_F|SEND_B|RECV_B|REDUCE_GRAD|F|B|I|W)(\d*)(?:@(\d+))?$")

    @staticmethod
    def parse(text: str) -> "Action":
        m = Action._PATTERN.match(text.strip())
        if m is None:
            raise ValueError(f"cannot parse schedule action {text!r}")
        stage, op, mb, peer = m.groups()
        return Action(int(stage), Op(op), int(mb) if mb != "" else None, int(peer) if peer is not None else None)


Schedule = Dict[int, List[Action]]  # rank -> actions


def linear_topology(num_stages: int) -> Dict[int, List[int]]:
    """Stage s feeds stage s+1 and nothing else."""
    return {s: ([s + 1] if s + 1 < num_stages else []) for s in range(num_stages)}


def _sources(dests: Dict[int, List[int]]) -> Dict[int, List[int]]:
    src: Dict[int, List[int]] = {s: [] for s in dests}
    for s, ds in dests.items():
        for d in ds:
            src.setdefault(d, []).append(s)
    return src


class ScheduleDeadlock(RuntimeError):
    pass


def add_send_recv(
    compute: Schedule,
    stage_to_rank: Callable[[int], int],
    num_stages: int,
    dests: Optional[Dict[int, List[int]]] = None,
) -> Schedule:
    """Inserts SEND/RECV actions into per-rank compute lists.

    All ranks are replayed in lock step; a rank takes its next compute action only when the actions it depends on
    were taken in an earlier round.  A transfer's SEND and its RECV are appended to both ranks in the same round,
    so every pair of ranks sees its transfers in the same order and there is one global order all ranks respect:
    the resulting lists cannot deadlock on an in-order transport.  Transfers between two stages of the same rank
    need no communication and get no actions.  Raises :class:`ScheduleDeadlock` if the compute order itself is
    infeasible.
    """
    dests = dests if dests is not None else linear_topology(num_stages)
    srcs = _sources(dests)
    ranks = sorted(compute.keys())
    out: Schedule = {r: [] for r in ranks}
    ptr = {r: 0 for r in ranks}
    done = set()

    def ready(a: Action) -> bool:
        if a.op == Op.F:
            return all((s, "F", a.mb) in done for s in srcs.get(a.stage, []))
        if a.op in (Op.B, Op.I):
            if (a.stage, "F", a.mb) not in done:
                return False
            return all((d, "BI", a.mb) in done for d in dests.get(a.stage, []))
        if a.op == Op.W:
            return (a.stage, "BI", a.mb) in done
        return True

    while any(ptr[r] < len(compute[r]) for r in ranks):
        newly = []
        for r in ranks:
            if ptr[r] >= len(compute[r]):
                continue
            a = compute[r][ptr[r]]
            if not a.op.is_compute:
                out[r].append(a)
                ptr[r] += 1
                newly.append(None)
                continue
            if not ready(a):
                continue
            out[r].append(a)
            ptr[r] += 1
            if a.op == Op.F:
                newly.append((a.stage, "F", a.mb))
                remote = [d for d in dests.get(a.stage, []) if stage_to_rank(d) != r]
                if remote:
                    out[r].append(Action(a.stage, Op.SEND_F, a.mb))
                    for d in sorted(remote):
                        out[stage_to_rank(d)].append(Action(d, Op.RECV_F, a.mb, peer=a.stage))
            elif a.op in (Op.B, Op.I):
                newly.append((a.stage, "BI", a.mb))
                remote = [s for s in srcs.get(a.stage, []) if stage_to_rank(s) != r]
                if remote:
                    out[r].append(Action(a.stage, Op.SEND_B, a.mb))
                    for s in sorted(remote):
                        out[stage_to_rank(s)].append(Action(s, Op.RECV_B, a.mb, peer=a.stage))
            else:
                newly.append((a.stage, "W", a.mb))
        if not newly:
            stuck = {r: compute[r][ptr[r]] for r in ranks if ptr[r] < len(compute[r])}
            raise ScheduleDeadlock(f"schedule cannot make progress; next actions per rank: {stuck}")
        done.update(x for x in newly if x is not None)
    return out


def validate(compute: Schedule, num_stages: int, n_microbatches: int, stage_to_rank: Callable[[int], int]) -> None:
    """Checks that every (stage, microbatch) has exactly one F and one B (or one I and one W) on the right rank."""
    seen: Dict[tuple, int] = {}
    for r, actions in compute.items():
        for a in actions:
            if not a.op.is_compute:
                continue
            if stage_to_rank(a.stage) != r:
                raise ValueError(f"action {a} scheduled on rank {r} but its stage lives on rank {stage_to_rank(a.stage)}")
            key = (a.stage, a.op, a.mb)
            seen[key] = seen.get(key, 0) + 1
    for s in range(num_stages):
        for mb in range(n_microbatches):
            if seen.get((s, Op.F, mb), 0) != 1:
                raise ValueError(f"stage {s} microbatch {mb}: expected exactly one F, got {seen.get((s, Op.F, mb), 0)}")
            nb = seen.get((s, Op.B, mb), 0)
            ni = seen.get((s, Op.I, mb), 0)
            nw = seen.get((s, Op.W, mb), 0)
            if nb + ni == 0:
                continue  # forward-only schedule
            if not ((nb == 1 and ni == 0 and nw == 0) or (nb == 0 and ni == 1 and nw == 1)):
                raise ValueError(f"stage {s} microbatch {mb}: B={nb} I={ni} W={nw}")


def dump_csv(schedule: Schedule, path: str) -> None:
    """One row per rank, one action per cell (same idea as upstream's schedule CSV)."""
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        for r in sorted(schedule):
            w.writerow([str(a) for a in schedule[r]])


def load_csv(path: str) -> Schedule:
    out: Schedule = {}
    with open(path, newline="") as f:
        for r, row in enumerate(csv.reader(f)):
            out[r] = [Action.parse(cell) for cell in row if cell.strip()]
    return out


def format_schedule(schedule: Schedule) -> str:
    return "\n".join(f"rank {r}: " + " ".join(str(a) for a in schedule[r]) for r in sorted(schedule))
