"""Happens-before check of the peer-memory protocols (``gt_b200.utils.hb_check`` on the programs of ``gt_b200.parallel.protocol_model``)."""
import os
import re

import pytest

from gt_b200.parallel import protocol_model as pm
from gt_b200.utils.hb_check import ProtocolTrace, check

GRIDS = [(1, 2), (2, 1), (2, 2), (4, 2), (2, 4), (8, 1), (1, 8)]


def test_checker_on_hand_written_programs():
    # publish / consume through a channel: ordered
    tr = ProtocolTrace(2)
    tr.write(0, 0, "b", 1); tr.signal(0, "c", (0, 1)); tr.signal(1, "c", (0, 1)); tr.wait(1, "c", (0, 1), 0); tr.read(1, 0, "b", 1)
    assert not check(tr).violations
    # the consumer does not wait: the read may come first
    tr = ProtocolTrace(2)
    tr.write(0, 0, "b", 1); tr.read(1, 0, "b", 1)
    assert [v.kind for v in check(tr).violations] == ["read-before-write"]
    # ordering through a third rank: 0 -> 2 -> 1
    tr = ProtocolTrace(3)
    tr.write(0, 0, "b", 1); tr.signal(0, "a", (0, 2))
    tr.signal(2, "a", (0, 2)); tr.wait(2, "a", (0, 2), 0); tr.signal(2, "z", (1, 2))
    tr.signal(1, "z", (1, 2)); tr.wait(1, "z", (1, 2), 2); tr.read(1, 0, "b", 1)
    assert not check(tr).violations
    # the owner overwrites while the reader has not said that it is done
    tr = ProtocolTrace(2)
    tr.write(0, 0, "b", 1); tr.signal(0, "c", (0, 1)); tr.write(0, 0, "b", 2)
    tr.signal(1, "c", (0, 1)); tr.wait(1, "c", (0, 1), 0); tr.read(1, 0, "b", 1)
    kinds = {v.kind for v in check(tr).violations}
    assert kinds and kinds <= {"write-while-read", "read-before-write", "wrong-version"}
    # two writers of one location without an order between them
    tr = ProtocolTrace(2)
    tr.write(0, 0, "b", 1); tr.write(1, 0, "b", 2)
    assert [v.kind for v in check(tr).violations] == ["write-write"]
    # a wait before the first signal of the waiting rank needs nothing (epoch 0)
    tr = ProtocolTrace(2)
    tr.wait(0, "c", (0, 1), 1)
    rep = check(tr)
    assert rep.completed and not rep.expired


@pytest.mark.parametrize("grid", GRIDS)
def test_fused_step_is_race_free(grid):
    for layers in (1, 2, 3, 4):
        for kw in (dict(), dict(eval_after=True), dict(recompute=True), dict(recompute=True, eval_after=True)):
            rep = check(pm.fused_step_trace(grid[0], grid[1], layers, steps=3, **kw))
            assert rep.completed and not rep.violations and not rep.expired and not any(rep.status), (grid, layers, kw, pm.describe(rep))


def test_single_buffering_is_caught():
    rep = check(pm.fused_step_trace(2, 2, 3, steps=2, copies=1))
    assert any(v.kind == "write-while-read" and v.buf[1] == "fb_x" for v in rep.violations)
    rep = check(pm.fused_step_trace(2, 1, 2, steps=1, copies=1))
    assert {v.buf[1] for v in rep.violations} == {"fb_x", "fb_dxc"}
    # a row group alone is ordered layer by layer by its payload exchange (every member waits for every member): one copy would do
    assert not check(pm.fused_step_trace(1, 2, 3, steps=2, copies=1)).violations
    assert not check(pm.barrier_collective_trace(4, 6)).violations
    assert check(pm.barrier_collective_trace(4, 6, copies=1)).violations


def test_begin_step_barriers_are_what_protects_the_restart_of_the_alternation():
    # odd depth + recomputation + an evaluation pass: the last use before a step and the first use of the step take the same copy,
    # and nothing but the barriers of begin_step orders them
    kw = dict(recompute=True, eval_after=True)
    assert check(pm.fused_step_trace(2, 2, 3, steps=2, begin_barriers=False, **kw)).violations
    assert not check(pm.fused_step_trace(2, 2, 3, steps=2, begin_barriers=True, **kw)).violations


def test_lost_signal_expires_the_waits_on_that_peer_and_nobody_blocks():
    rep = check(pm.fused_step_trace(2, 2, 3, steps=2), drop={(1, "pay0", 2)})
    assert rep.completed
    assert {(r, chan, peer) for r, _, chan, peer in rep.expired} == {(0, "pay0", 1), (1, "pay0", 1)}
    assert rep.status[:2] == [101, 101] and rep.status[2:] == [0, 0]          # index of the silent peer within its row group
    assert any(v.kind == "read-before-write" and v.buf[1] == "fb_pay" for v in rep.violations)       # what the expired wait no longer guarantees
    worst = check(pm.fused_step_trace(2, 2, 3, steps=2), drop={(1, "pay0", 2)}, cascade=True)
    assert worst.completed and set(rep.expired) <= set(worst.expired) and len(worst.expired) > len(rep.expired)
    rep = check(pm.fused_step_trace(4, 2, 4, steps=2), drop={(5, "barrier_world", 2)})
    assert rep.completed and rep.status == [105] * 8 and not rep.violations


def test_stopped_rank_leaves_no_rank_blocked():
    rep = check(pm.fused_step_trace(2, 2, 2, steps=2), die={3: 60})
    assert rep.completed and rep.expired
    assert all(peer == 3 for _, _, _, peer in rep.expired)
    assert all(s >= 100 for s in rep.status[:3]) and rep.status[3] == 0


def test_model_names_the_staging_kinds_and_channels_of_the_source():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = open(os.path.join(root, "gt_b200", "parallel", "fused_layer.py")).read()
    model = open(os.path.join(root, "gt_b200", "parallel", "protocol_model.py")).read()
    kinds_src = set(re.findall(r'staging\([^"]*"(fb_\w+)"\)', src))
    kinds_model = set(re.findall(r'staging\("(fb_\w+)"', model))
    assert kinds_src == kinds_model == {"fb_x", "fb_pay", "fb_dpay", "fb_dxc", "fb_dxr"}
    chans_src = set(re.findall(r"comm\.(\w+)\.signal\(\)", src))
    chans_model = set(re.findall(r'tr\.signal\(r, "(\w+?)%d"', model))
    assert chans_src == chans_model == {"x_col", "x_row", "pay", "dpay", "dx_col", "dx_row"}


def test_cli(capsys):
    assert pm.main(["--grid", "2", "2", "--layers", "2", "--steps", "2"]) == 0
    assert "violations 0" in capsys.readouterr().out
    assert pm.main(["--grid", "2", "2", "--layers", "2", "--copies", "1"]) == 1
    assert pm.main(["--grid", "2", "1", "--layers", "2", "--drop", "1", "x_col0", "1"]) == 1
    assert "expired: rank 0" in capsys.readouterr().out


def _all_orders(trace):
    """Brute force over every interleaving of a small trace that respects the waits: for each pair of conflicting accesses (same
    location, different ranks, at least one write) the set of relative orders that occur; ``None`` if some interleaving gets stuck."""
    world = trace.world
    progs = trace.prog
    orders = {}
    stuck = [False]

    def rec(pcs, counts, published, seen):
        if all(pcs[r] == len(progs[r]) for r in range(world)):
            return
        moved = False
        for r in range(world):
            if pcs[r] == len(progs[r]):
                continue
            op, a, b, _, _ = progs[r][pcs[r]]
            c2, p2, s2 = counts, published, seen
            if op == "wait":
                if published[b].get(a, 0) < counts[r].get(a, 0):
                    continue
            elif op == "signal":
                k = counts[r].get(a, 0) + 1
                c2 = [dict(c) for c in counts]; c2[r][a] = k
                p2 = [dict(p) for p in published]; p2[r][a] = k
            else:
                me = (r, pcs[r], op, (a, b))
                for other in seen:
                    if other[3] == me[3] and other[0] != r and "write" in (op, other[2]):
                        orders.setdefault(frozenset((other[:2], me[:2])), set()).add((other[:2], me[:2]))
                s2 = seen + (me,)
            moved = True
            n = list(pcs); n[r] += 1
            rec(tuple(n), c2, p2, s2)
        if not moved:
            stuck[0] = True

    rec(tuple([0] * world), [dict() for _ in range(world)], [dict() for _ in range(world)], ())
    return None if stuck[0] else orders


def test_checker_agrees_with_brute_force_on_random_small_programs():
    """The vector-clock verdict of one execution against the definition of a race (two conflicting accesses that occur in both orders
    over all interleavings), on random programs of two or three ranks: it reports something if and only if a race exists."""
    pytest.importorskip("hypothesis")
    from hypothesis import assume, given, settings, strategies as st
    bufs, chans = ["p", "q"], ["c", "d"]

    def op_strategy(world):
        return st.one_of(
            st.tuples(st.just("write"), st.integers(0, world - 1), st.sampled_from(bufs)),
            st.tuples(st.just("read"), st.integers(0, world - 1), st.sampled_from(bufs)),
            st.tuples(st.just("signal"), st.sampled_from(chans)),
            st.tuples(st.just("wait"), st.sampled_from(chans), st.integers(0, world - 1)))

    @settings(max_examples=400, deadline=None, derandomize=True)
    @given(st.integers(2, 3).flatmap(lambda w: st.tuples(st.just(w), st.lists(st.lists(op_strategy(w), min_size=1, max_size=4), min_size=w, max_size=w))))
    def run(case):
        world, programs = case
        members = tuple(range(world))
        tr = ProtocolTrace(world)
        for r, ops in enumerate(programs):
            for op in ops:
                if op[0] == "write":
                    tr.write(r, op[1], op[2], None)
                elif op[0] == "read":
                    tr.read(r, op[1], op[2], None)
                elif op[0] == "signal":
                    tr.signal(r, op[1], members)
                else:
                    tr.wait(r, op[1], members, op[2])
        orders = _all_orders(tr)
        assume(orders is not None)                           # programs that can get stuck are another matter (expiring waits)
        racy = any(len(v) == 2 for v in orders.values())
        rep = check(tr, require_writes=False)
        assert rep.completed and not rep.expired
        assert bool(rep.violations) == racy, (programs, rep.violations, orders)

    run()


def test_recorded_byte_ranges_conflict_exactly_when_they_overlap():
    pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st
    from gt_b200.utils.hb_check import trace_from_logs
    rng = st.tuples(st.integers(0, 40), st.integers(1, 24))

    @settings(max_examples=300, deadline=None, derandomize=True)
    @given(rng, rng, st.booleans())
    def run(a, b, synchronised):
        logs = [[("write", 0, a[0], a[1])], [("read", 0, b[0], b[1])]]
        if synchronised:                                     # rank 1 waits for rank 0's signal before it reads
            logs[0].append(("signal", 1000, (0, 1)))
            logs[1] = [("signal", 1000, (0, 1)), ("wait", 1000, 0)] + logs[1]
        overlap = a[0] < b[0] + b[1] and b[0] < a[0] + a[1]
        rep = check(trace_from_logs(logs), require_writes=False)
        assert bool(rep.violations) == (overlap and not synchronised), (a, b, synchronised, rep.violations)

    run()
