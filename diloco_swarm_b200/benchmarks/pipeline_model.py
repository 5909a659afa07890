"""Timing model of a training step: replay the real routing table and per-rank plans with stage times.

    python -m diloco_swarm_b200.benchmarks.pipeline_model --stages 2 --replicas 4 --micro-batches 32 \
        --cap 8 --fwd-ms 3.9,3.6 --bwd-ms 7.8,7.3 --xfer-ms 0.07 --routing uniform --steps 200

The routing function and the plan generator are the ones the trainer uses (parallel/schedule.py), so
the model sees the same stochastic wiring, the same in-flight cap and the same order of operations
on every rank; only the durations are inputs.  Every rank runs its plan in order; an operation
starts when the rank is free and its input has arrived (the producer's end time plus the transfer
time).  The output is the distribution of the step time over seeded steps, the share of the step
that the busiest and the average rank spend computing, and the tokens per second that follow.

It answers the questions the reference's notebooks answer by hand (notebooks/3.0-results.ipynb) and
two that they do not: what uniform routing costs against balanced routing at a given number of
replicas (the straggler replica sets the step time), and how many microbatches have to be in
flight before the pipeline stops waiting.  It needs no GPU.
"""
from __future__ import annotations

import argparse
import json
import statistics
from typing import Dict, List, Optional, Sequence

from ..parallel import schedule as S


def step_time(plans: Dict[int, List[S.Op]], num_stages: int, fwd: Sequence[float], bwd: Sequence[float],
              xfer: float, speed: Optional[Sequence[float]] = None) -> Dict[str, float]:
    """Replay one step.  ``fwd[s]`` / ``bwd[s]``: time of one microbatch's forward / backward on stage
    ``s``; ``xfer``: time for an activation or gradient tile to reach the neighbouring stage;
    ``speed[r]``: relative speed of rank ``r`` (its durations are divided by it).
    Returns the makespan and the busy time of every rank."""
    world = len(plans)
    pos = {r: 0 for r in plans}
    free = {r: 0.0 for r in plans}
    busy = {r: 0.0 for r in plans}
    arrived: Dict[tuple, float] = {}              # (direction, mb, destination rank) -> arrival time
    progressed = True
    while progressed:
        progressed = False
        for r, ops in plans.items():
            st = r % num_stages
            while pos[r] < len(ops):
                op = ops[pos[r]]
                ready = 0.0
                if op.kind in (S.FWD, S.FWD_BWD) and op.prev >= 0:
                    key = ("f", op.mb, r)
                    if key not in arrived:
                        break
                    ready = arrived[key]
                if op.kind == S.BWD and op.next >= 0:
                    key = ("b", op.mb, r)
                    if key not in arrived:
                        break
                    ready = arrived[key]
                dur = fwd[st] if op.kind == S.FWD else bwd[st] if op.kind == S.BWD else fwd[st] + bwd[st]
                if speed is not None:
                    dur /= speed[r]
                start = max(free[r], ready)
                free[r] = start + dur
                busy[r] += dur
                if op.kind == S.FWD and op.next >= 0:
                    arrived[("f", op.mb, op.next)] = free[r] + xfer
                if op.kind in (S.BWD, S.FWD_BWD) and op.prev >= 0:
                    arrived[("b", op.mb, op.prev)] = free[r] + xfer
                pos[r] += 1
                progressed = True
    if any(pos[r] < len(plans[r]) for r in plans):
        raise RuntimeError("the plans do not complete: a rank waits for a message nobody sends")
    return {"makespan": max(free.values()) if world else 0.0, "busy": busy}


def simulate(stages: int, replicas: int, micro_batches: int, cap: int, fwd: Sequence[float], bwd: Sequence[float],
             xfer: float = 0.0, routing: str = "uniform", steps: int = 100, seed: int = 0,
             tail_ms: float = 0.0, speed: Optional[Sequence[float]] = None,
             weights: Optional[Sequence[float]] = None) -> Dict[str, float]:
    """Step-time statistics over ``steps`` seeded routings.  ``tail_ms`` is added to every step
    (optimiser, gradient or outer synchronisation, metrics).  ``speed``: relative speed per rank
    (heterogeneous replicas); ``weights``: routing weights per rank for ``routing = "weighted"``
    (default: the speeds)."""
    if routing == "weighted" and weights is None:
        weights = speed
    world = stages * replicas
    times, peak_util, mean_util, worst_share = [], [], [], []
    for step in range(1, steps + 1):
        path = S.route(seed, step, stages, world, micro_batches, mode=routing, weights=weights)
        plans = {r: S.plan(path, world, r, cap) for r in range(world)}
        out = step_time(plans, stages, fwd, bwd, xfer, speed)
        t = out["makespan"] + tail_ms
        times.append(t)
        busy = list(out["busy"].values())
        peak_util.append(max(busy) / t)
        mean_util.append(sum(busy) / len(busy) / t)
        last = [sum(1 for op in plans[r] if op.kind == S.FWD_BWD) for r in range(world) if r % stages == stages - 1]
        worst_share.append(max(last) / (micro_batches / replicas))
    return {"step_ms_mean": statistics.mean(times), "step_ms_median": statistics.median(times),
            "step_ms_p90": sorted(times)[int(0.9 * (len(times) - 1))], "step_ms_max": max(times),
            "busiest_rank_utilisation": statistics.mean(peak_util), "mean_rank_utilisation": statistics.mean(mean_util),
            "busiest_last_stage_replica_vs_even_share": statistics.mean(worst_share)}


def _floats(text: str, n: int) -> List[float]:
    v = [float(x) for x in text.split(",")]
    if len(v) == 1:
        v = v * n
    if len(v) != n:
        raise SystemExit(f"expected 1 or {n} comma-separated values, got {text!r}")
    return v


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--stages", type=int, default=2)
    ap.add_argument("--replicas", type=int, default=4)
    ap.add_argument("--micro-batches", type=int, default=32)
    ap.add_argument("--cap", type=int, default=8, help="max_micro_batches: microbatches in flight per rank")
    ap.add_argument("--fwd-ms", default="3.7", help="forward time of one microbatch per stage (one value or one per stage)")
    ap.add_argument("--bwd-ms", default="7.4", help="backward time of one microbatch per stage")
    ap.add_argument("--xfer-ms", type=float, default=0.07, help="activation / gradient transfer time between stages")
    ap.add_argument("--tail-ms", type=float, default=2.0, help="per-step work after the pipeline (optimiser, syncs)")
    ap.add_argument("--routing", default="uniform", choices=list(S.ROUTING_MODES))
    ap.add_argument("--speed", default="", help="relative speed per rank, comma separated (default: all 1)")
    ap.add_argument("--weights", default="", help="routing weights per rank for --routing weighted (default: the speeds)")
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tokens-per-micro-batch", type=int, default=16 * 1024)
    a = ap.parse_args()
    world = a.stages * a.replicas
    speed = _floats(a.speed, world) if a.speed else None
    weights = _floats(a.weights, world) if a.weights else None
    out = simulate(a.stages, a.replicas, a.micro_batches, a.cap, _floats(a.fwd_ms, a.stages), _floats(a.bwd_ms, a.stages),
                   a.xfer_ms, a.routing, a.steps, a.seed, a.tail_ms, speed, weights)
    out["tokens_per_s_at_mean_step"] = a.micro_batches * a.tokens_per_micro_batch / (out["step_ms_mean"] / 1e3)
    out["config"] = {k: v for k, v in vars(a).items()}
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
