import collections

import numpy as np
import pytest

from diloco_swarm_b200.parallel import schedule as S


def test_route_is_deterministic_and_respects_stages():
    p1 = S.route(7, 3, 3, 9, 24)
    p2 = S.route(7, 3, 3, 9, 24)
    assert np.array_equal(p1, p2)
    assert not np.array_equal(p1, S.route(7, 4, 3, 9, 24))        # changes with the step
    assert not np.array_equal(p1, S.route(8, 3, 3, 9, 24))        # and with the seed
    for s in range(3):
        assert set(p1[:, s]) <= {r for r in range(9) if r % 3 == s}
    # first stage: round-robin chunks as in the reference's BatchSampler
    assert list(p1[:, 0]) == [[0, 3, 6][mb % 3] for mb in range(24)]


def test_route_is_roughly_uniform():
    c = collections.Counter(int(S.route(1, t, 2, 8, 32)[i, 1]) for t in range(200) for i in range(32))
    assert set(c) == {1, 3, 5, 7}
    assert max(c.values()) / min(c.values()) < 1.15


def test_route_skips_dead_replicas():
    alive = [True] * 8
    alive[3] = alive[4] = False
    p = S.route(1, 1, 2, 8, 64, alive)
    assert 3 not in p and 4 not in p
    with pytest.raises(RuntimeError):
        S.route(1, 1, 2, 2, 4, [True, False])


@pytest.mark.parametrize("stages,world,M,cap", [(1, 1, 4, 1), (2, 2, 8, 1), (2, 4, 16, 3), (3, 9, 30, 2), (4, 8, 32, 4)])
def test_plan_is_complete_and_causal(stages, world, M, cap):
    path = S.route(5, 2, stages, world, M)
    plans = {r: S.plan(path, world, r, cap) for r in range(world)}
    fwd_seen = collections.defaultdict(set)
    for r, ops in plans.items():
        st = r % stages
        inflight = 0
        for op in ops:
            assert path[op.mb, st] == r
            if op.kind == S.FWD:
                inflight += 1
                assert inflight <= cap or st == stages - 1
                fwd_seen[r].add(op.mb)
            elif op.kind == S.BWD:
                assert op.mb in fwd_seen[r]          # backward only after its own forward
                inflight -= 1
            else:
                assert st == stages - 1
        assert inflight == 0
    # every microbatch runs forward and backward exactly once on every stage
    for mb in range(M):
        for st in range(stages):
            ops = [o for o in plans[int(path[mb, st])] if o.mb == mb]
            kinds = sorted(o.kind for o in ops)
            assert kinds == ([S.FWD_BWD] if st == stages - 1 else [S.FWD, S.BWD])


def _simulate(plans, world, forward_only=False):
    """Replay the plans with in-order point-to-point channels; returns True if every rank finishes."""
    pos = {r: 0 for r in range(world)}
    sent = collections.defaultdict(list)        # (src, dst, direction) -> queue of mbs
    progressed = True
    while progressed:
        progressed = False
        for r in range(world):
            while pos[r] < len(plans[r]):
                op = plans[r][pos[r]]
                if op.kind in (S.FWD, S.FWD_BWD) and op.prev >= 0:
                    q = sent[(op.prev, r, "f")]
                    if not q or q[0] != op.mb:
                        break
                    q.pop(0)
                if op.kind == S.BWD and op.next >= 0:
                    q = sent[(op.next, r, "b")]
                    if not q or q[0] != op.mb:
                        break
                    q.pop(0)
                if op.kind == S.FWD and op.next >= 0:
                    sent[(r, op.next, "f")].append(op.mb)
                if op.kind in (S.BWD, S.FWD_BWD) and op.prev >= 0 and not forward_only:
                    sent[(r, op.prev, "b")].append(op.mb)
                pos[r] += 1
                progressed = True
    return all(pos[r] == len(plans[r]) for r in range(world))


@pytest.mark.parametrize("stages,world,M,cap", [(2, 2, 8, 1), (2, 4, 32, 4), (2, 8, 32, 2), (3, 9, 27, 3), (4, 8, 32, 1)])
def test_plans_do_not_deadlock_on_fifo_channels(stages, world, M, cap):
    for step in range(1, 6):
        path = S.route(11, step, stages, world, M)
        plans = {r: S.plan(path, world, r, cap) for r in range(world)}
        assert _simulate(plans, world)
        fplans = {r: S.plan(path, world, r, cap, forward_only=True) for r in range(world)}
        assert all(o.kind == S.FWD for ops in fplans.values() for o in ops)
        assert _simulate(fplans, world, forward_only=True)


def test_micro_batch_key_matches_reference_naming():
    assert S.micro_batch_key(0, [0, 2]) == (0, 1)
    assert S.micro_batch_key(1, [0, 2]) == (2, 1)
    assert S.micro_batch_key(5, [0, 2]) == (2, 3)


def test_balanced_routing_gives_equal_shares_and_uniform_marginals():
    counts = collections.Counter()
    for step in range(300):
        p = S.route(9, step, 2, 8, 32, mode="balanced")
        per = collections.Counter(p[:, 1].tolist())
        assert set(per.values()) == {8}                       # 32 microbatches over 4 replicas
        counts[int(p[5, 1])] += 1
    assert max(counts.values()) / min(counts.values()) < 1.6   # one microbatch still lands anywhere
    p = S.route(9, 1, 3, 9, 10, mode="balanced")               # 10 over 3: shares differ by at most one
    for s in (1, 2):
        v = collections.Counter(p[:, s].tolist()).values()
        assert max(v) - min(v) <= 1


def test_random_worlds_masks_and_modes_never_deadlock():
    """Property test: for random stage counts, replica counts, microbatch counts, in-flight caps, routing
    modes and live masks (at least one live replica per stage), every rank's plan completes when replayed
    over in-order channels, dead ranks get no work and the cap holds."""
    hyp = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st

    @st.composite
    def worlds(draw):
        stages = draw(st.integers(1, 4))
        replicas = draw(st.integers(1, 4))
        world = stages * replicas
        alive = [True] * world
        for s in range(stages):
            dead = draw(st.lists(st.integers(0, replicas - 1), max_size=replicas - 1, unique=True))
            for k in dead:
                alive[s + k * stages] = False
        return (stages, world, alive, draw(st.integers(1, 24)), draw(st.integers(1, 5)),
                draw(st.sampled_from(["uniform", "balanced"])), draw(st.integers(0, 1000)), draw(st.integers(1, 50)))

    @settings(max_examples=150, deadline=None)
    @given(worlds())
    def check(w):
        stages, world, alive, M, cap, mode, seed, step = w
        path = S.route(seed, step, stages, world, M, alive, mode=mode)
        assert all(alive[int(r)] for r in path.reshape(-1))
        plans = {r: S.plan(path, world, r, cap) for r in range(world)}
        for r in range(world):
            if not alive[r]:
                assert plans[r] == []
            inflight = 0
            for op in plans[r]:
                if op.kind == S.FWD:
                    inflight += 1
                    assert inflight <= cap
                elif op.kind == S.BWD:
                    inflight -= 1
        assert _simulate(plans, world)

    check()


def test_weighted_routing_follows_the_weights():
    """Hops land on a replica in proportion to its weight; dead or zero-weight replicas get nothing; the
    first stage keeps its round-robin chunks; without weights the mode draws uniformly."""
    stages, world, M = 2, 8, 64
    w = [1, 1, 1, 1, 1, 3, 1, 0]                      # stage-1 replicas are ranks 1, 3, 5, 7
    hits = collections.Counter()
    for step in range(200):
        p = S.route(3, step, stages, world, M, mode="weighted", weights=w)
        assert p[:, 0].tolist() == [2 * (i % 4) for i in range(M)]
        hits.update(p[:, 1].tolist())
    total = sum(hits.values())
    assert hits[7] == 0 and set(hits) == {1, 3, 5}
    assert abs(hits[5] / total - 0.6) < 0.02 and abs(hits[1] / total - 0.2) < 0.02
    alive = [True] * world
    alive[5] = False
    p = S.route(3, 1, stages, world, M, alive, mode="weighted", weights=w)
    assert set(p[:, 1].tolist()) <= {1, 3}
    flat = collections.Counter()
    for step in range(200):
        flat.update(S.route(3, step, stages, world, M, mode="weighted")[:, 1].tolist())
    assert max(flat.values()) / min(flat.values()) < 1.15
    assert (S.route(3, 7, stages, world, M, mode="weighted", weights=w) ==
            S.route(3, 7, stages, world, M, mode="weighted", weights=w)).all()


def test_check_plans_accepts_real_plans_and_names_what_is_wrong_with_broken_ones():
    import dataclasses
    for stages, world, M, cap, mode in ((1, 2, 6, 1, "uniform"), (2, 4, 16, 3, "uniform"), (3, 9, 27, 2, "balanced"),
                                        (4, 8, 32, 4, "uniform")):
        path = S.route(3, 5, stages, world, M, mode=mode)
        plans = {r: S.plan(path, world, r, cap) for r in range(world)}
        S.check_plans(path, plans, cap)
        fplans = {r: S.plan(path, world, r, cap, forward_only=True) for r in range(world)}
        S.check_plans(path, fplans, cap, forward_only=True)
    path = S.route(3, 5, 2, 4, 16)
    good = {r: S.plan(path, 4, r, 3) for r in range(4)}

    def broken(change):
        plans = {r: list(ops) for r, ops in good.items()}
        change(plans)
        with pytest.raises(S.PlanError) as e:
            S.check_plans(path, plans, 3)
        return str(e.value)

    assert "expected" in broken(lambda p: p[0].pop())                                    # a backward is missing
    first_bwd = next(i for i, o in enumerate(good[0]) if o.kind == S.BWD)
    assert "before its forward" in broken(lambda p: p[0].insert(0, p[0].pop(first_bwd)))
    assert "routing" in broken(lambda p: p[0].__setitem__(0, dataclasses.replace(p[0][0], next=0)))
    assert "limit" in broken(lambda p: p[0].sort(key=lambda o: o.kind))                  # all forwards first: over the cap
    # two last-stage ranks each wait for a tile that its sender has queued behind the other one's
    last = [r for r in (1, 3)]
    def swap_first_two(p):
        for r in last:
            if len(p[r]) >= 2:
                p[r][0], p[r][1] = p[r][1], p[r][0]
    msg = broken(swap_first_two)
    assert "deadlock" in msg or "expected" in msg


def test_busiest_replica_loads_and_the_split_that_follows_them():
    """Uniform wiring: the first stage's replicas serve M / R each (roots are dealt round-robin), a later
    stage's busiest replica clearly more; the balanced split then moves a block from the last stage to the
    first when there are four replicas per stage, and not when there is one."""
    from diloco_swarm_b200.models.gpt2 import balanced_split
    loads = S.busiest_replica_loads(42, 2, 8, 32, "uniform")
    assert loads[0] == 8.0 and 9.5 < loads[1] < 11.5
    assert S.busiest_replica_loads(42, 2, 8, 32, "balanced") == [8.0, 8.0]
    assert S.busiest_replica_loads(42, 2, 2, 32, "uniform") == [32.0, 32.0]
    assert balanced_split(12, 2, 768, 50304) == [8, 4]
    assert balanced_split(12, 2, 768, 50304, loads) == [9, 3]
    assert balanced_split(12, 1, 768, 50304) == [12]
    for n, st, d in ((24, 4, 1024), (36, 8, 1280), (48, 3, 1600), (4, 2, 128)):
        c = balanced_split(n, st, d, 50304)
        assert sum(c) == n and len(c) == st and min(c) >= 1


def test_plans_with_stage_costs_stay_consistent():
    """Per-stage costs change the order of a rank's operations, never their set; the plans of all ranks
    still pass the consistency check."""
    path = S.route(7, 3, 2, 8, 32)
    for costs in (None, ([0.3, 1.2], [0.7, 2.4]), ([2.9, 2.4], [6.1, 5.1])):
        kw = {} if costs is None else {"cost_f": costs[0], "cost_b": costs[1]}
        plans = {r: S.plan(path, 8, r, 8, **kw) for r in range(8)}
        S.check_plans(path, plans, 8)
        assert sorted((o.kind, o.mb) for o in plans[1]) == sorted((o.kind, o.mb) for o in S.plan(path, 8, 1, 8))
