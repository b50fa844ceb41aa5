"""Properties of the schedule generators, checked on CPU with the simulator."""
import os

import pytest

from pippy_b200.schedules import actions as A
from pippy_b200.schedules import generators as G
from pippy_b200.schedules import simulator as S
from pippy_b200.schedules.actions import Action, Op


def _check(schedule, P, v, n):
    s2r = lambda s: s % P
    A.validate(schedule, P * v, n, s2r)
    full = A.add_send_recv(schedule, s2r, P * v)
    for r, acts in full.items():
        sends = [a for a in acts if a.op in (Op.SEND_F, Op.SEND_B)]
        recvs = [a for a in acts if a.op in (Op.RECV_F, Op.RECV_B)]
        assert len(sends) == len(recvs) or P > 1
    cost = {Op.F: 1.0 / v, Op.B: 2.0 / v, Op.I: 1.0 / v, Op.W: 1.0 / v}
    return S.simulate(full, s2r, P * v, cost)


@pytest.mark.parametrize("P,n", [(2, 4), (4, 8), (4, 3), (8, 32)])
def test_gpipe_and_1f1b_have_the_analytic_bubble(P, n):
    for sched in (G.gpipe(P, n), G.one_f_one_b(P, n), G.one_f_one_b(P, n, reference_warmup=True)):
        r = _check(sched, P, 1, n)
        assert abs(r.max_bubble - S.ideal_bubble(P, n)) < 1e-9


def test_1f1b_warmup_counts_match_reference_formula():
    P, n = 4, 8
    ref = G.one_f_one_b(P, n, reference_warmup=True)
    txt = G.one_f_one_b(P, n)
    for r in range(P):
        lead_ref = next(i for i, a in enumerate(ref[r]) if a.op == Op.B)
        lead_txt = next(i for i, a in enumerate(txt[r]) if a.op == Op.B)
        assert lead_ref == min(n, 2 * (P - r - 1)) + 1
        assert lead_txt == min(n, P - r - 1) + 1
    r_ref, r_txt = _check(ref, P, 1, n), _check(txt, P, 1, n)
    assert r_ref.peak_in_flight[0] > r_txt.peak_in_flight[0]


@pytest.mark.parametrize("P,v,n", [(2, 2, 4), (4, 2, 8), (8, 2, 32), (1, 2, 4)])
def test_interleaved_bubble_and_warmup(P, v, n):
    sched = G.interleaved_1f1b(P, v, n)
    r = _check(sched, P, v, n)
    assert abs(r.max_bubble - S.ideal_bubble(P, n, v)) < 1e-9
    for rank in range(P):
        first_b = next(i for i, a in enumerate(sched[rank]) if a.op == Op.B)
        assert first_b == min((v - 1) * P + 2 * ((P - 1) - rank), v * n) + 1
        assert {a.stage for a in sched[rank]} == {rank + k * P for k in range(v)}


def test_interleaved_rejects_bad_microbatch_count():
    with pytest.raises(ValueError):
        G.interleaved_1f1b(4, 2, 6)
    with pytest.raises(ValueError):
        G.zero_bubble(4, 2, 6)


@pytest.mark.parametrize("P,v,n", [(4, 1, 8), (4, 2, 8), (8, 2, 32), (2, 1, 4)])
def test_zero_bubble_beats_1f1b_and_bounds_memory(P, v, n):
    zb = _check(G.zero_bubble(P, v, n), P, v, n)
    base = _check(G.interleaved_1f1b(P, v, n) if v > 1 else G.one_f_one_b(P, n), P, v, n)
    assert zb.makespan < base.makespan
    assert zb.max_bubble < base.max_bubble
    for r in range(P):
        assert zb.peak_in_flight[r] <= (v - 1) * P + (P - 1 - r) + 1


def test_looped_bfs_order():
    sched = G.looped_bfs(2, 2, 3)
    assert [str(a) for a in sched[0][:6]] == ["0F0", "0F1", "0F2", "2F0", "2F1", "2F2"]
    assert [str(a) for a in sched[0][6:]] == ["2B0", "2B1", "2B2", "0B0", "0B1", "0B2"]
    _check(sched, 2, 2, 3)


def _deep_costed_order(P, v, n):
    # the benchmark's case: measured-looking costs with a heavy last stage, up to 8 more microbatches in flight
    S = P * v
    cost = {s: (5.5, 6.1, 4.9) for s in range(S)}
    cost[S - 1] = (6.9, 7.3, 5.8)
    return G.tuned_zero_bubble_costed(P, v, n, cost, {s: 0.4 for s in range(S - 1)},
                                      extra_in_flight=(0, 1, 2, 4, 6, 8), pending_w=(P, 2 * P))


@pytest.mark.parametrize("P,v,n,make", [(4, 2, 8, G.zero_bubble), (8, 2, 32, _deep_costed_order)])
def test_send_recv_pairing_is_consistent_between_neighbours(P, v, n, make):
    order = make(P, v, n)
    A.validate(order, P * v, n, lambda s: s % P)
    full = A.add_send_recv(order, lambda s: s % P, P * v)
    # the k-th transfer a rank sends to a peer is the k-th that peer receives from it
    for r in range(P):
        for peer in range(P):
            sent = [(a.op, a.stage, a.mb) for a in full[r]
                    if a.op in (Op.SEND_F, Op.SEND_B)
                    and ((a.stage + (1 if a.op == Op.SEND_F else -1)) % P == peer)]
            got = [(a.op, a.peer, a.mb) for a in full[peer]
                   if a.op in (Op.RECV_F, Op.RECV_B) and (a.peer % P == r)]
            assert [(s[1], s[2]) for s in sent] == [(g[1], g[2]) for g in got]


def test_infeasible_order_is_reported():
    bad = {0: [Action(0, Op.B, 0), Action(0, Op.F, 0)], 1: [Action(1, Op.F, 0), Action(1, Op.B, 0)]}
    with pytest.raises(A.ScheduleDeadlock):
        A.add_send_recv(bad, lambda s: s, 2)


def test_csv_roundtrip_and_parse(tmp_path):
    sched = A.add_send_recv(G.zero_bubble(2, 2, 4), lambda s: s % 2, 4)
    path = os.path.join(tmp_path, "s.csv")
    A.dump_csv(sched, path)
    assert A.load_csv(path) == sched
    assert Action.parse("3RECV_F7@2") == Action(3, Op.RECV_F, 7, 2)
    assert str(Action(1, Op.REDUCE_GRAD)) == "1REDUCE_GRAD"
    with pytest.raises(ValueError):
        Action.parse("F3")


def test_skip_connection_topology_in_comm_planning():
    # stage 0 feeds stages 1 and 3
    dests = {0: [1, 3], 1: [2], 2: [3], 3: []}
    full = A.add_send_recv(G.gpipe(4, 2), lambda s: s, 4, dests)
    assert Action(3, Op.RECV_F, 0, peer=0) in full[3] and Action(3, Op.RECV_F, 0, peer=2) in full[3]
    assert Action(0, Op.RECV_B, 1, peer=3) in full[0] and Action(0, Op.RECV_B, 1, peer=1) in full[0]
    S.simulate(full, lambda s: s, 4, dests=dests)


def test_reduce_grad_placed_after_last_weight_action():
    sched = G.with_reduce_grad(G.zero_bubble(2, 1, 4))
    for r, acts in sched.items():
        idx = [i for i, a in enumerate(acts) if a.op == Op.REDUCE_GRAD]
        assert len(idx) == 1
        assert all(a.op not in (Op.W, Op.B) for a in acts[idx[0] + 1:])


def test_chrome_trace_of_simulated_and_measured_timelines(tmp_path):
    import json

    from pippy_b200.schedules import measured_trace, simulated_trace, simulate, write_chrome_trace, zero_bubble

    P, v, n = 4, 2, 8
    sched = zero_bubble(P, v, n)
    res = simulate(sched, lambda s: s % P, P * v, cost={Op.F: 2.0, Op.I: 3.0, Op.W: 2.0, Op.B: 5.0})
    events = simulated_trace(res)
    assert len(events) == sum(len(t) for t in res.timeline.values())
    assert {e["tid"] for e in events} == set(range(P))
    # rows never overlap in time: a rank runs one action at a time
    for r in range(P):
        rows = sorted((e["ts"], e["ts"] + e["dur"]) for e in events if e["tid"] == r)
        assert all(a[1] <= b[0] + 1e-6 for a, b in zip(rows, rows[1:]))
    stats = {"timeline": [("F(s0,mb0)", 0.0, 0.001), ("B(s0,mb0)", 0.002, 0.004)]}
    ev = measured_trace(stats, rank=3)
    assert ev[1]["ts"] == pytest.approx(2000.0) and ev[1]["dur"] == pytest.approx(2000.0) and ev[1]["tid"] == 3
    path = tmp_path / "trace.json"
    write_chrome_trace(str(path), events + ev, {r: f"rank {r}" for r in range(P)})
    data = json.loads(path.read_text())
    assert len(data["traceEvents"]) == len(events) + len(ev) + P


@pytest.mark.parametrize("P,n", [(2, 2), (2, 8), (3, 5), (4, 4), (4, 16), (8, 8), (8, 32)])
def test_v_shaped_zero_bubble_is_valid_and_beats_interleaved(P, n):
    placement = G.v_placement(P)
    assert placement[0] == placement[2 * P - 1] == 0 and placement[P - 1] == placement[P] == P - 1
    cost = {Op.F: 2.0, Op.I: 3.0, Op.W: 2.0, Op.B: 5.0}
    for extra in (0, 3):
        for mpw in (1, P, 4 * P):
            sched = G.zero_bubble_placed(P, placement, n, extra, mpw)       # never deadlocks, whatever the limits
            A.validate(sched, 2 * P, n, lambda s: placement[s])
            S.simulate(sched, lambda s: placement[s], 2 * P, cost=cost)
    tuned = G.tuned_zero_bubble_placed(P, placement, n)
    A.validate(tuned, 2 * P, n, lambda s: placement[s])
    res = S.simulate(tuned, lambda s: placement[s], 2 * P, cost=cost)
    if n % P == 0:
        inter = S.simulate(G.interleaved_1f1b(P, 2, n), lambda s: s % P, 2 * P, cost=cost)
        assert res.makespan <= inter.makespan
    # both ends of the model on rank 0: the comm plan has no link between rank 0 and rank P-1 other than neighbours
    with_comm = A.add_send_recv(tuned, lambda s: placement[s], 2 * P)
    peer_ranks = {placement[a.peer] for a in with_comm[0] if a.op.is_comm and a.peer is not None}
    assert peer_ranks <= {1}


def test_placement_errors():
    with pytest.raises(ValueError):
        G.zero_bubble_placed(2, {0: 0, 1: 1, 3: 0}, 4)
    with pytest.raises(ValueError):
        G.zero_bubble_placed(2, {0: 0, 1: 0, 2: 0, 3: 0}, 4)


@pytest.mark.parametrize("P,v", [(2, 2), (4, 2), (8, 2), (4, 1)])
def test_costed_zero_bubble_is_valid_and_no_slower_than_the_fixed_guess(P, v):
    """The order built from per-stage costs (a heavy last stage, I : W unlike 3 : 2, a transfer latency) runs every
    action once, respects the dependencies, and replayed on those same costs is not slower than the default order."""
    from pippy_b200.schedules import generators as g
    from pippy_b200.schedules.actions import Op, validate

    n, S = 16, P * v
    cost = {s: (6.0, 9.5, 5.0) for s in range(S)}
    cost[S - 1] = (8.0, 11.0, 7.0)
    lat = 0.3

    def replay(sched):
        finish, clock, ptr = {}, {r: 0.0 for r in sched}, {r: 0 for r in sched}
        moved = True
        while moved:
            moved = False
            for r in sched:
                while ptr[r] < len(sched[r]):
                    a = sched[r][ptr[r]]
                    s, m = a.stage, a.mb
                    if a.op == Op.F:
                        deps = [(s - 1, "F", m)] if s > 0 else []
                    elif a.op == Op.I:
                        deps = [(s, "F", m)] + ([(s + 1, "I", m)] if s < S - 1 else [])
                    else:
                        deps = [(s, "I", m)]
                    if any(d not in finish for d in deps):
                        break
                    start = max([clock[r]] + [finish[d] + (lat if d[0] % P != r else 0.0) for d in deps])
                    end = start + cost[s]["FIW".index(a.op.value)]
                    finish[(s, a.op.value, m)] = clock[r] = end
                    ptr[r] += 1
                    moved = True
        assert all(ptr[r] == len(sched[r]) for r in sched)
        return max(clock.values())

    fixed = g.zero_bubble(P, v, n)
    costed = g.tuned_zero_bubble_costed(P, v, n, cost, lat)
    validate(costed, S, n, lambda s: s % P)
    assert replay(costed) <= replay(fixed) * 1.001
    # the V-shaped placement goes through the same generator
    if v == 2:
        placed = g.zero_bubble_costed(P, 2, n, cost, lat, placement=g.v_placement(P))
        validate(placed, S, n, lambda s: g.v_placement(P)[s])
