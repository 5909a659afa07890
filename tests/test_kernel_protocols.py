"""The barrier protocols of the warp-specialised kernels (attention backward and forward, the persistent GEMM),
replayed on the CPU with random latencies: every role finishes (no deadlock), no shared buffer is overwritten
under a reader and every reader finds the data version it expects (no hazard); and each wait that is left out
on purpose is noticed."""
import random

import pytest

from diloco_swarm_b200.utils.attention_protocol import IMPLIED, MUTATIONS, run_attention_bwd
from diloco_swarm_b200.utils.protocol_sim import Barrier, Deadlock, Hazard, Sim


def _items(rng):
    return [rng.randint(1, 8) for _ in range(rng.randint(1, 10))]


def test_barrier_parity_semantics():
    b = Barrier("b", 2)
    assert b.done(1) and not b.done(0)          # a fresh barrier: the phase "before the first" counts as done
    b.arrive()
    assert not b.done(0)
    b.arrive()
    assert b.done(0) and not b.done(1)


def test_protocol_is_deadlock_and_hazard_free():
    for seed in range(300):
        rng = random.Random(seed)
        t = run_attention_bwd(_items(rng), rng)
        assert t > 0
    # the shapes that matter most: only single-step items (a hand-over between items on every step), one item
    for seed in range(50):
        rng = random.Random(1000 + seed)
        run_attention_bwd([1] * rng.randint(1, 12), rng)
        run_attention_bwd([rng.randint(1, 8)], rng)


@pytest.mark.parametrize("drop", MUTATIONS)
def test_a_missing_wait_is_noticed(drop):
    seen = 0
    for seed in range(200):
        rng = random.Random(seed)
        try:
            run_attention_bwd(_items(rng), rng, drop=drop)
        except (Hazard, Deadlock):
            seen += 1
    assert seen > 0, f"leaving out {drop} went unnoticed in 200 random runs"


@pytest.mark.parametrize("drop", IMPLIED)
def test_an_implied_wait_can_go_without_harm(drop):
    for seed in range(200):
        rng = random.Random(seed)
        run_attention_bwd(_items(rng), rng, drop=drop)


def test_sim_reports_a_deadlock():
    sim = Sim()
    never = Barrier("never", 1)

    def role():
        yield ("wait", never, 0)
    sim.add_role("r", role())
    with pytest.raises(Deadlock):
        sim.run()


# ---------------------------------------------------------------- forward attention and the GEMM kernels
from diloco_swarm_b200.utils.attention_protocol import FWD_IMPLIED, FWD_MUTATIONS, run_attention_fwd  # noqa: E402
from diloco_swarm_b200.utils import gemm_protocol  # noqa: E402


def test_forward_protocol_is_deadlock_and_hazard_free():
    for seed in range(300):
        rng = random.Random(seed)
        run_attention_fwd(_items(rng), rng)
    for seed in range(50):
        rng = random.Random(2000 + seed)
        run_attention_fwd([1] * rng.randint(1, 12), rng)


@pytest.mark.parametrize("drop", FWD_MUTATIONS)
def test_forward_a_missing_wait_is_noticed(drop):
    seen = 0
    for seed in range(200):
        rng = random.Random(seed)
        try:
            run_attention_fwd(_items(rng), rng, drop=drop)
        except (Hazard, Deadlock):
            seen += 1
    assert seen > 0, f"leaving out {drop} went unnoticed in 200 random runs"


@pytest.mark.parametrize("drop", FWD_IMPLIED)
def test_forward_an_implied_wait_can_go_without_harm(drop):
    for seed in range(200):
        rng = random.Random(seed)
        run_attention_fwd(_items(rng), rng, drop=drop)


def test_gemm_protocol_is_deadlock_and_hazard_free():
    for seed in range(200):
        rng = random.Random(seed)
        gemm_protocol.run_gemm(rng.randint(1, 7), rng.randint(1, 24), rng.choice([2, 3, 4, 6]), rng)


@pytest.mark.parametrize("drop", gemm_protocol.MUTATIONS)
def test_gemm_a_missing_wait_is_noticed(drop):
    seen = 0
    for seed in range(200):
        rng = random.Random(seed)
        try:
            gemm_protocol.run_gemm(rng.randint(2, 7), rng.randint(1, 24), rng.choice([2, 3, 4, 6]), rng, drop=drop)
        except (Hazard, Deadlock):
            seen += 1
    assert seen > 0, f"leaving out {drop} went unnoticed in 200 random runs"


def test_step_time_model_of_the_attention_backward():
    """benchmarks/attention_bwd_model: with the measured latencies the model gives the step time seen on the
    GPU (2.4-2.6 us), and shorter reloads or cheaper MMA issue shorten it while faster row algebra hardly does."""
    from diloco_swarm_b200.benchmarks.attention_bwd_model import MEASURED, step_time
    items = [8, 5, 5, 2, 2, 7, 7, 4, 4, 1, 1]
    base = step_time(items, dict(MEASURED))
    assert 2300 < base < 2800
    assert step_time(items, {**MEASURED, "tma": 600.0}) < 0.93 * base
    assert step_time(items, {**MEASURED, "t_issue": 26.0, "t_mma": 30.0}) < 0.9 * base
    assert step_time(items, {**MEASURED, "compute": 600.0}) > 0.95 * base
