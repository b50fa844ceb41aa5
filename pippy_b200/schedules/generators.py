"""Pure generators of per-rank compute orders for every supported schedule.

Stage ``s`` of an interleaved (multi-stage-per-rank) pipeline lives on rank ``s % P`` (reference
pippy/_PipelineStage.py:129-136), so a rank's local stages are ``rank + k*P``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

from .actions import Action, Op, Schedule


def gpipe(P: int, n_mb: int, backward: bool = True) -> Schedule:
    """Fill-drain: all forwards, then all backwards in microbatch order (reference PipelineSchedule.py:279-355)."""
    out: Schedule = {}
    for r in range(P):
        acts = [Action(r, Op.F, m) for m in range(n_mb)]
        if backward:
            acts += [Action(r, Op.B, m) for m in range(n_mb)]
        out[r] = acts
    return out


def one_f_one_b(P: int, n_mb: int, backward: bool = True, reference_warmup: bool = False) -> Schedule:
    """1F1B. ``reference_warmup`` uses the reference's 2*(P-r-1) warm-up forwards
    (PipelineSchedule.py:379-387) instead of the textbook P-r-1; the bubble is the same, the reference form keeps
    twice as many activations in flight."""
    out: Schedule = {}
    for r in range(P):
        if not backward:
            out[r] = [Action(r, Op.F, m) for m in range(n_mb)]
            continue
        depth = (P - r - 1) * (2 if reference_warmup else 1)
        warm = min(n_mb, depth)
        acts: List[Action] = []
        f = b = 0
        for _ in range(warm):
            acts.append(Action(r, Op.F, f))
            f += 1
        while f < n_mb:
            acts.append(Action(r, Op.F, f))
            f += 1
            acts.append(Action(r, Op.B, b))
            b += 1
        while b < n_mb:
            acts.append(Action(r, Op.B, b))
            b += 1
        out[r] = acts
    return out


def looped_bfs(P: int, v: int, n_mb: int, backward: bool = True) -> Schedule:
    """Breadth-first over a rank's local stages: every microbatch through local stage 0, then stage 1, ...;
    backward in reverse stage order (reference PipelineSchedule.py:517-569)."""
    out: Schedule = {}
    for r in range(P):
        stages = [r + k * P for k in range(v)]
        acts = [Action(s, Op.F, m) for s in stages for m in range(n_mb)]
        if backward:
            acts += [Action(s, Op.B, m) for s in reversed(stages) for m in range(n_mb)]
        out[r] = acts
    return out


def _interleaved_orders(P: int, v: int, n_mb: int, r: int):
    """Forward and backward visiting orders of rank r: microbatches advance in rounds of P per local stage."""
    total = v * n_mb
    f_count = [0] * v
    b_count = [0] * v
    f_seq, b_seq = [], []
    for step in range(total):
        k = (step // P) % v
        f_seq.append((r + k * P, f_count[k]))
        f_count[k] += 1
        kb = v - 1 - ((step // P) % v)
        b_seq.append((r + kb * P, b_count[kb]))
        b_count[kb] += 1
    return f_seq, b_seq


def interleaved_1f1b(P: int, v: int, n_mb: int, backward: bool = True) -> Schedule:
    """Interleaved 1F1B with ``v`` stages per rank (reference PipelineSchedule.py:572-778, warm-up math :623-640)."""
    if n_mb % P != 0:
        raise ValueError(
            f"Interleaved 1F1B requires the number of microbatches ({n_mb}) to be a multiple of the pipeline "
            f"group size ({P})"
        )
    out: Schedule = {}
    total = v * n_mb
    for r in range(P):
        f_seq, b_seq = _interleaved_orders(P, v, n_mb, r)
        if not backward:
            out[r] = [Action(s, Op.F, m) for s, m in f_seq]
            continue
        warm = min((v - 1) * P + 2 * ((P - 1) - r), total)
        acts: List[Action] = [Action(s, Op.F, m) for s, m in f_seq[:warm]]
        b = 0
        for i in range(warm, total):
            s, m = f_seq[i]
            acts.append(Action(s, Op.F, m))
            s, m = b_seq[b]
            acts.append(Action(s, Op.B, m))
            b += 1
        while b < total:
            s, m = b_seq[b]
            acts.append(Action(s, Op.B, m))
            b += 1
        out[r] = acts
    return out


def zero_bubble(
    P: int,
    v: int,
    n_mb: int,
    max_pending_w: Optional[int] = None,
    extra_in_flight: int = 0,
    cost_f: int = 2,
    cost_i: int = 3,
    cost_w: int = 2,
) -> Schedule:
    """Zero-bubble schedule with the backward split into I (input grads) and W (weight grads).

    Built by list scheduling on a timeline with costs F:I:W (default 2:3:2, a transformer layer whose input-gradient
    pass carries the attention backward): each rank visits forwards and input-gradient passes in the
    interleaved-1F1B orders, always prefers a ready I, then a ready F while fewer than
    ``(v-1)*P + (P-1-r) + 1 + extra_in_flight`` microbatch-stages are in flight, and fills every remaining gap
    with the oldest deferred W (``max_pending_w`` bounds how many weight-gradient passes may be parked, and with
    them the activations they keep alive).  With v == 1 this is the ZB-H1 shape; v > 1 corresponds to
    upstream's interleaved zero-bubble schedule.
    """
    if v > 1 and n_mb % P != 0:
        raise ValueError(
            f"interleaved zero-bubble requires the number of microbatches ({n_mb}) to be a multiple of the "
            f"pipeline group size ({P})"
        )
    S = P * v
    total = v * n_mb
    if max_pending_w is None:
        max_pending_w = max(2 * P, 4)
    f_seq, i_seq = {}, {}
    for r in range(P):
        f_seq[r], i_seq[r] = _interleaved_orders(P, v, n_mb, r)
    cap = {r: (v - 1) * P + (P - 1 - r) + 1 + extra_in_flight for r in range(P)}
    fp = {r: 0 for r in range(P)}
    ip = {r: 0 for r in range(P)}
    wq: Dict[int, List] = {r: [] for r in range(P)}
    in_flight = {r: 0 for r in range(P)}
    busy_until = {r: 0 for r in range(P)}
    finish: Dict[tuple, int] = {}  # (stage, kind, mb) -> completion time
    out: Schedule = {r: [] for r in range(P)}
    t = 0
    remaining = P * total * 3
    guard = 0
    while remaining > 0:
        guard += 1
        if guard > 100 * P * total + 1000:
            raise RuntimeError("zero-bubble list scheduling failed to converge")
        for r in range(P):
            if busy_until[r] > t:
                continue
            choice = None
            if ip[r] < total:
                s, m = i_seq[r][ip[r]]
                dep_ok = finish.get((s, "F", m), 1 << 60) <= t and (
                    s == S - 1 or finish.get((s + 1, "I", m), 1 << 60) <= t
                )
                if dep_ok:
                    choice = ("I", s, m)
            if choice is None and len(wq[r]) > max_pending_w:
                choice = ("W",) + wq[r][0]
            if choice is None and fp[r] < total and in_flight[r] < cap[r]:
                s, m = f_seq[r][fp[r]]
                if s == 0 or finish.get((s - 1, "F", m), 1 << 60) <= t:
                    choice = ("F", s, m)
            if choice is None and wq[r]:
                choice = ("W",) + wq[r][0]
            if choice is None:
                continue
            kind, s, m = choice
            if kind == "F":
                fp[r] += 1
                in_flight[r] += 1
                dur = cost_f
                out[r].append(Action(s, Op.F, m))
            elif kind == "I":
                ip[r] += 1
                in_flight[r] -= 1
                wq[r].append((s, m))
                dur = cost_i
                out[r].append(Action(s, Op.I, m))
            else:
                wq[r].pop(0)
                dur = cost_w
                out[r].append(Action(s, Op.W, m))
            finish[(s, kind, m)] = t + dur
            busy_until[r] = t + dur
            remaining -= 1
        t += 1
    return out


def zero_bubble_costed(
    P: int,
    v: int,
    n_mb: int,
    cost: Dict[int, tuple],
    comm_latency: float = 0.0,
    max_pending_w: Optional[int] = None,
    extra_in_flight: int = 0,
    placement: Optional[Dict[int, int]] = None,
    return_makespan: bool = False,
):
    """Zero-bubble order from MEASURED per-stage costs: ``cost[s] = (forward, input-gradient, weight-gradient)``
    durations of one microbatch on stage ``s``, in any common unit.  Same policy as :func:`zero_bubble` (a ready I
    first, then a forward while the in-flight limit allows, weight gradients in the gaps), but on a continuous
    event-driven timeline, so that a heavier stage (the one with the LM head and the loss) and an I : W ratio that
    differs from the 3 : 2 guess shift the order instead of showing up as idle time.  A value produced on another
    rank becomes usable ``comm_latency`` after its producer ends; a dict ``{s: seconds}`` gives the transfer time of
    the boundary between stages ``s`` and ``s + 1`` (both directions) when boundaries carry different amounts.  With ``placement`` (stage -> rank) the forward and
    input-gradient orders are per stage, nearest the loss first, as in :func:`zero_bubble_placed`."""
    S = P * v if placement is None else len(placement)
    where = (lambda s: s % P) if placement is None else (lambda s: placement[s])
    if placement is None and v > 1 and n_mb % P != 0:
        raise ValueError(
            f"interleaved zero-bubble requires the number of microbatches ({n_mb}) to be a multiple of the "
            f"pipeline group size ({P})"
        )
    if sorted(cost) != list(range(S)):
        raise ValueError(f"cost must give (F, I, W) for stages 0..{S - 1}")
    if max_pending_w is None:
        max_pending_w = max(2 * P, 4)
    local = {r: sorted((s for s in range(S) if where(s) == r), reverse=True) for r in range(P)}
    wrap = placement is None
    if wrap:
        f_seq, i_seq = {}, {}
        for r in range(P):
            f_seq[r], i_seq[r] = _interleaved_orders(P, v, n_mb, r)
        fp = {r: 0 for r in range(P)}
        ip = {r: 0 for r in range(P)}
        cap_rank = {r: (v - 1) * P + (P - 1 - r) + 1 + extra_in_flight for r in range(P)}
        in_flight_rank = {r: 0 for r in range(P)}
    else:
        next_f = {s: 0 for s in range(S)}
        next_i = {s: 0 for s in range(S)}
        cap_stage = {s: min(n_mb, S - s + extra_in_flight) for s in range(S)}
        in_flight_stage = {s: 0 for s in range(S)}
    wq: Dict[int, List] = {r: [] for r in range(P)}
    free_at = {r: 0.0 for r in range(P)}
    left = {r: 3 * n_mb * len(local[r]) for r in range(P)}
    finish: Dict[tuple, float] = {}
    out: Schedule = {r: [] for r in range(P)}
    INF = float("inf")

    def latency(boundary):
        return comm_latency.get(boundary, 0.0) if isinstance(comm_latency, dict) else comm_latency

    def ready_at(key, consumer_rank, boundary):
        t = finish.get(key)
        if t is None:
            return INF
        return t + (latency(boundary) if where(key[0]) != consumer_rank else 0.0)

    def f_ready(s, m, r):
        return 0.0 if s == 0 else ready_at((s - 1, "F", m), r, s - 1)

    def i_ready(s, m, r):
        t = ready_at((s, "F", m), r, s)
        return t if s == S - 1 else max(t, ready_at((s + 1, "I", m), r, s))

    blocked = set()  # ranks waiting for a producer that nobody has scheduled yet
    while any(left.values()):
        runnable = [q for q in range(P) if left[q] and q not in blocked]
        if not runnable:
            # every rank waits for a producer that no rank may start (the two limits can block each other)
            raise RuntimeError("zero-bubble list scheduling is stuck: the in-flight and pending limits deadlock")
        r = min(runnable, key=lambda q: (free_at[q], q))
        t = free_at[r]
        choice = None
        waits = []  # times at which something this rank could do becomes ready
        # 1. a ready input-gradient pass
        if wrap:
            if ip[r] < len(i_seq[r]):
                s, m = i_seq[r][ip[r]]
                ta = i_ready(s, m, r)
                if ta <= t:
                    choice = ("I", s, m)
                else:
                    waits.append(ta)
        else:
            cands = []
            for s in local[r]:
                m = next_i[s]
                if m < n_mb:
                    ta = i_ready(s, m, r)
                    if ta <= t:
                        cands.append((m, -s, s))
                    else:
                        waits.append(ta)
            if cands:
                m, _, s = min(cands)
                choice = ("I", s, m)
        # 2. too many parked weight gradients
        if choice is None and len(wq[r]) > max_pending_w:
            choice = ("W",) + wq[r][0]
        # 3. a ready forward within the in-flight limit
        if choice is None:
            if wrap:
                if fp[r] < len(f_seq[r]) and in_flight_rank[r] < cap_rank[r]:
                    s, m = f_seq[r][fp[r]]
                    ta = f_ready(s, m, r)
                    if ta <= t:
                        choice = ("F", s, m)
                    else:
                        waits.append(ta)
            else:
                for s in local[r]:
                    m = next_f[s]
                    if m < n_mb and in_flight_stage[s] < cap_stage[s]:
                        ta = f_ready(s, m, r)
                        if ta <= t:
                            choice = ("F", s, m)
                            break
                        waits.append(ta)
        # 4. fill the gap with the oldest parked weight gradient
        if choice is None and wq[r]:
            choice = ("W",) + wq[r][0]
        if choice is None:
            # idle until the next known arrival; with none known, sleep until some rank schedules an action (only
            # that can make one of this rank's producers known)
            nxt = [w for w in waits if t < w < INF]
            if nxt:
                free_at[r] = min(nxt)
            else:
                blocked.add(r)
            continue
        for q in blocked:
            free_at[q] = max(free_at[q], t)
        blocked.clear()
        kind, s, m = choice
        cf, ci, cw = cost[s]
        if kind == "F":
            if wrap:
                fp[r] += 1
                in_flight_rank[r] += 1
            else:
                next_f[s] += 1
                in_flight_stage[s] += 1
            dur = cf
            out[r].append(Action(s, Op.F, m))
        elif kind == "I":
            if wrap:
                ip[r] += 1
                in_flight_rank[r] -= 1
            else:
                next_i[s] += 1
                in_flight_stage[s] -= 1
            wq[r].append((s, m))
            dur = ci
            out[r].append(Action(s, Op.I, m))
        else:
            wq[r].pop(0)
            dur = cw
            out[r].append(Action(s, Op.W, m))
        finish[(s, kind, m)] = t + dur
        free_at[r] = t + dur
        left[r] -= 1
    if return_makespan:
        return out, max(free_at.values())
    return out


def tuned_zero_bubble_costed(P: int, v: int, n_mb: int, cost: Dict[int, tuple], comm_latency: float = 0.0,
                             extra_in_flight: tuple = (0, 1, 2), pending_w: Optional[tuple] = None,
                             placement: Optional[Dict[int, int]] = None, slack: float = 0.003) -> Schedule:
    """Replays a few settings of the two limits of :func:`zero_bubble_costed` and keeps, among those within
    ``slack`` of the shortest makespan, the one that holds the fewest microbatches in flight."""
    pending_w = pending_w or (P, 2 * P, 4 * P)
    tried = []
    for extra in extra_in_flight:
        for mpw in pending_w:
            try:
                sched, span = zero_bubble_costed(P, v, n_mb, cost, comm_latency, mpw, extra, placement, True)
            except RuntimeError:
                continue  # this pair of limits blocks itself; the others are still candidates
            tried.append((span, extra, mpw, sched))
    if not tried:
        raise RuntimeError("no setting of the zero-bubble limits produced a schedule")
    best = min(t[0] for t in tried)
    close = [t for t in tried if t[0] <= best * (1.0 + slack)]
    return min(close, key=lambda t: (t[1], t[2], t[0]))[3]


def with_reduce_grad(schedule: Schedule) -> Schedule:
    """Appends a REDUCE_GRAD action right after the last weight-producing action (B or W) of every stage."""
    out: Schedule = {}
    for r, acts in schedule.items():
        last: Dict[int, int] = {}
        for idx, a in enumerate(acts):
            if a.op in (Op.B, Op.W):
                last[a.stage] = idx
        new: List[Action] = []
        for idx, a in enumerate(acts):
            new.append(a)
            for s, li in last.items():
                if li == idx:
                    new.append(Action(s, Op.REDUCE_GRAD))
        out[r] = new
    return out


def v_placement(P: int) -> Dict[int, int]:
    """Stage -> rank map of the V shape: rank r holds stage r on the way down and stage 2P-1-r on the way up, so
    the first and the last stage share rank 0 and the turn (stages P-1, P) is a local hand-over on rank P-1."""
    return {s: (s if s < P else 2 * P - 1 - s) for s in range(2 * P)}


def zero_bubble_placed(
    P: int,
    placement: Dict[int, int],
    n_mb: int,
    extra_in_flight: int = 0,
    max_pending_w: Optional[int] = None,
    cost_f: int = 2,
    cost_i: int = 3,
    cost_w: int = 2,
) -> Schedule:
    """Zero-bubble schedule for an arbitrary stage -> rank placement, by greedy list scheduling on a timeline.

    No per-rank order is assumed (the wrap-around generator above takes its orders from interleaved 1F1B): whenever
    a rank is free it takes, in this order of preference, a ready input-gradient pass (oldest microbatch first, the
    stage nearest the loss first), a parked weight-gradient pass if more than ``max_pending_w`` are parked, a ready
    forward (the stage nearest the loss first, so that microbatches reach the loss and start their backward early)
    while that STAGE holds fewer than ``S - s + extra_in_flight`` microbatches (the 1F1B bound per stage: a limit per
    rank can fill up with early-stage microbatches and starve the stage they must pass next), and otherwise the
    oldest parked weight gradient.  With ``v_placement(P)`` this gives the V-shaped zero-bubble schedule (upstream's ZBV,
    torch/distributed/pipelining/schedules.py:2811-3000): at costs F = I = W it has no bubble beyond the fill, and
    rank 0 holds both the embedding and the LM head.
    """
    S = len(placement)
    if sorted(placement) != list(range(S)):
        raise ValueError("placement must map stages 0..S-1")
    local: Dict[int, List[int]] = {r: sorted((s for s in placement if placement[s] == r), reverse=True) for r in range(P)}
    if any(not local[r] for r in range(P)):
        raise ValueError("every rank needs at least one stage")
    cap = {s: min(n_mb, S - s + extra_in_flight) for s in range(S)}
    if max_pending_w is None:
        max_pending_w = max(2 * P, 4)
    next_f = {s: 0 for s in range(S)}
    next_i = {s: 0 for s in range(S)}
    wq: Dict[int, List] = {r: [] for r in range(P)}
    in_flight = {s: 0 for s in range(S)}
    busy_until = {r: 0 for r in range(P)}
    finish: Dict[tuple, int] = {}
    out: Schedule = {r: [] for r in range(P)}
    remaining = 3 * S * n_mb
    t = 0
    guard = 0
    INF = 1 << 60
    while remaining > 0:
        guard += 1
        if guard > 200 * S * n_mb + 1000:
            raise RuntimeError("zero-bubble list scheduling failed to converge")
        for r in range(P):
            if busy_until[r] > t:
                continue
            choice = None
            ready_i = []
            for s in local[r]:
                m = next_i[s]
                if m < n_mb and finish.get((s, "F", m), INF) <= t and (s == S - 1 or finish.get((s + 1, "I", m), INF) <= t):
                    ready_i.append((m, -s, s))
            if ready_i:
                m, _, s = min(ready_i)
                choice = ("I", s, m)
            if choice is None and len(wq[r]) > max_pending_w:
                choice = ("W",) + wq[r][0]
            if choice is None:
                for s in local[r]:  # nearest the loss first
                    m = next_f[s]
                    if m < n_mb and in_flight[s] < cap[s] and (s == 0 or finish.get((s - 1, "F", m), INF) <= t):
                        choice = ("F", s, m)
                        break
            if choice is None and wq[r]:
                choice = ("W",) + wq[r][0]
            if choice is None:
                continue
            kind, s, m = choice
            if kind == "F":
                next_f[s] += 1
                in_flight[s] += 1
                dur = cost_f
                out[r].append(Action(s, Op.F, m))
            elif kind == "I":
                next_i[s] += 1
                in_flight[s] -= 1
                wq[r].append((s, m))
                dur = cost_i
                out[r].append(Action(s, Op.I, m))
            else:
                wq[r].pop(0)
                dur = cost_w
                out[r].append(Action(s, Op.W, m))
            finish[(s, kind, m)] = t + dur
            busy_until[r] = t + dur
            remaining -= 1
        t += 1
    return out


def tuned_zero_bubble_placed(
    P: int,
    placement: Dict[int, int],
    n_mb: int,
    cost_f: int = 2,
    cost_i: int = 3,
    cost_w: int = 2,
    extra_in_flight: tuple = (0, 2, 4),
    pending_w: Optional[tuple] = None,
    slack: float = 0.01,
) -> Schedule:
    """Greedy list scheduling is sensitive to its two limits, so a few settings are replayed on the cost model; of
    those within ``slack`` of the shortest makespan the one that holds the fewest activations is kept."""
    from .simulator import simulate

    S = len(placement)
    pending_w = pending_w or (P, 2 * P, 4 * P)
    cost = {Op.F: float(cost_f), Op.I: float(cost_i), Op.W: float(cost_w), Op.B: float(cost_i + cost_w)}
    tried = []
    for extra in extra_in_flight:
        for mpw in pending_w:
            sched = zero_bubble_placed(P, placement, n_mb, extra, mpw, cost_f, cost_i, cost_w)
            res = simulate(sched, lambda s: placement[s], S, cost=cost)
            tried.append((res.makespan, max(res.peak_in_flight.values()), max(res.peak_pending_w.values()), sched))
    shortest = min(t[0] for t in tried)
    close = [t for t in tried if t[0] <= shortest * (1.0 + slack)]
    return min(close, key=lambda t: (t[1], t[2], t[0]))[3]
