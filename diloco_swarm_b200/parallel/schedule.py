"""Seeded routing table and static per-rank plan (bindings of csrc/schedule.cpp).

Replaces three things in the reference at once: the sender-side
``random.choice`` (src/comm.py:91), receive-from-any-source (src/comm.py:67)
and the TCP-store step counter (src/world.py:73-94).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..ops import _build

FWD, BWD, FWD_BWD = 0, 1, 2

_lib = None


def _host():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(_build.build_host())
        lib.dsw_route.restype = ctypes.c_int
        lib.dsw_route.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int, ctypes.c_int,
                                  ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        lib.dsw_route_weighted.restype = ctypes.c_int
        lib.dsw_route_weighted.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.dsw_plan.restype = ctypes.c_int
        lib.dsw_plan.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                 ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                 ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
        lib.dsw_coll_touch_map.restype = ctypes.c_int
        lib.dsw_coll_touch_map.argtypes = [ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int,
                                           ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_void_p]
        _lib = lib
    return _lib


@dataclass(frozen=True)
class Op:
    kind: int        # FWD, BWD or FWD_BWD (last stage)
    mb: int          # global microbatch index within the step
    prev: int        # rank that serves this microbatch one stage earlier, or -1
    next: int        # rank that serves it one stage later, or -1


ROUTING_MODES = {"uniform": 0, "balanced": 1, "weighted": 2}


def route(seed: int, step: int, num_stages: int, world_size: int, num_micro_batches: int,
          alive: Optional[Sequence[bool]] = None, mode: str = "uniform",
          weights: Optional[Sequence[float]] = None) -> np.ndarray:
    """``path[mb, s]`` = rank serving microbatch ``mb`` at stage ``s``.

    ``uniform``: every hop is an independent uniform draw, as the reference's
    ``random.choice``.  ``balanced``: a seeded random permutation of an evenly
    filled assignment per stage; the replica of any one microbatch is still
    uniform, but replicas serve equal shares, so no replica is the straggler.
    ``weighted``: a hop lands on a replica with probability proportional to its
    entry in ``weights`` (one per rank, e.g. relative throughput), the SWARM
    paper's wiring rule; without weights it is the uniform draw."""
    path = np.empty((num_micro_batches, num_stages), dtype=np.int32)
    a = None
    if alive is not None:
        a = np.ascontiguousarray(np.asarray(alive, dtype=np.uint8))
        assert a.shape == (world_size,)
    if mode == "weighted":
        wv = None
        if weights is not None and len(weights) > 0:
            wv = np.ascontiguousarray(np.asarray(weights, dtype=np.float64))
            assert wv.shape == (world_size,), "routing weights: one per rank"
        rc = _host().dsw_route_weighted(seed & (2**64 - 1), step, num_stages, world_size, num_micro_batches,
                                        a.ctypes.data if a is not None else None,
                                        wv.ctypes.data if wv is not None else None, path.ctypes.data)
        if rc != 0:
            raise RuntimeError("routing failed: a stage has no live replica")
        return path
    rc = _host().dsw_route(seed & (2**64 - 1), step, num_stages, world_size, num_micro_batches,
                           a.ctypes.data if a is not None else None, ROUTING_MODES[mode], path.ctypes.data)
    if rc != 0:
        raise RuntimeError("routing failed: a stage has no live replica")
    return path


def busiest_replica_loads(seed: int, num_stages: int, world_size: int, num_micro_batches: int, mode: str = "uniform",
                          weights: Optional[Sequence[float]] = None, steps: int = 64) -> List[float]:
    """Microbatches per step that the busiest replica of each stage serves, averaged over the first ``steps``
    steps of the run's own routing.  Under uniform stochastic wiring the first stage is even (roots are dealt
    round-robin) and every later stage's busiest replica gets clearly more than M / R (about 10.5 of 32
    with four replicas); the step time follows the busiest replica, so the layer split weighs stages by this."""
    out = [0.0] * num_stages
    for step in range(1, steps + 1):
        path = route(seed, step, num_stages, world_size, num_micro_batches, None, mode=mode, weights=weights)
        for s in range(num_stages):
            out[s] += float(np.bincount(path[:, s], minlength=world_size).max())
    return [x / steps for x in out]


def plan(path: np.ndarray, world_size: int, rank: int, cap: int, forward_only: bool = False,
         cost_f: Optional[Sequence[float]] = None, cost_b: Optional[Sequence[float]] = None) -> List[Op]:
    """Ordered forward/backward ops of ``rank`` for one step."""
    M, S = path.shape
    path = np.ascontiguousarray(path, dtype=np.int32)
    max_ops = 2 * M + 1
    ops = np.empty((max_ops, 4), dtype=np.int32)
    cf = np.ascontiguousarray(cost_f, dtype=np.float32) if cost_f is not None else None
    cb = np.ascontiguousarray(cost_b, dtype=np.float32) if cost_b is not None else None
    n = _host().dsw_plan(S, world_size, M, cap, path.ctypes.data,
                         cf.ctypes.data if cf is not None else None,
                         cb.ctypes.data if cb is not None else None,
                         1 if forward_only else 0, rank, ops.ctypes.data, max_ops)
    if n < 0:
        raise RuntimeError(f"plan generation failed with code {n}")
    return [Op(int(k), int(m), int(p), int(nx)) for k, m, p, nx in ops[:n]]


def micro_batch_key(mb: int, first_stage_ranks: Sequence[int]) -> tuple:
    """(root_rank, local_micro_step) of microbatch ``mb`` in the reference's
    naming (src/utils.py:120-126): roots take microbatches round-robin and
    count their own from 1."""
    r0 = len(first_stage_ranks)
    return first_stage_ranks[mb % r0], mb // r0 + 1


class PlanError(RuntimeError):
    """The plans of a step are inconsistent: they would hang or compute something else than the step."""


def check_plans(path: np.ndarray, plans: Dict[int, List[Op]], cap: int, forward_only: bool = False) -> None:
    """Host-side check of one step's plans (the stand-in for a race detector on the pipeline): every
    microbatch runs exactly once per stage on the rank the routing names, a backward follows its own
    forward, no rank holds more than ``cap`` forwards in flight, neighbours agree on who sends what, and
    a replay over in-order point-to-point channels lets every rank finish (no deadlock).  Raises
    ``PlanError`` with the first violation.  The trainer runs it on every step with DSWARM_VERIFY_PLANS=1."""
    M, S_ = path.shape
    for r, ops in plans.items():
        st, inflight, seen = r % S_, 0, set()
        for op in ops:
            if int(path[op.mb, st]) != r:
                raise PlanError(f"rank {r} runs microbatch {op.mb}, which the routing gives to rank {int(path[op.mb, st])}")
            want_prev = int(path[op.mb, st - 1]) if st > 0 else -1
            want_next = int(path[op.mb, st + 1]) if st + 1 < S_ else -1
            if (op.prev, op.next) != (want_prev, want_next):
                raise PlanError(f"rank {r}, microbatch {op.mb}: neighbours {(op.prev, op.next)}, routing says {(want_prev, want_next)}")
            if op.kind == FWD:
                inflight += 1
                seen.add(op.mb)
                if inflight > cap and st != S_ - 1 and not forward_only:
                    raise PlanError(f"rank {r} holds {inflight} forwards in flight, the limit is {cap}")
            elif op.kind == BWD:
                if op.mb not in seen:
                    raise PlanError(f"rank {r} runs the backward of microbatch {op.mb} before its forward")
                inflight -= 1
            elif st != S_ - 1:
                raise PlanError(f"rank {r} of stage {st} has a fused forward-backward, which only the last stage runs")
    for mb in range(M):
        for st in range(S_):
            kinds = sorted(o.kind for o in plans.get(int(path[mb, st]), []) if o.mb == mb)
            want = [FWD] if forward_only else ([FWD_BWD] if st == S_ - 1 else [FWD, BWD])
            if kinds != want:
                raise PlanError(f"microbatch {mb} at stage {st}: operations {kinds}, expected {want}")
    # replay on in-order channels
    pos = {r: 0 for r in plans}
    queues: Dict[tuple, List[int]] = {}
    progressed = True
    while progressed:
        progressed = False
        for r, ops in plans.items():
            while pos[r] < len(ops):
                op = ops[pos[r]]
                need = None
                if op.kind in (FWD, FWD_BWD) and op.prev >= 0:
                    need = (op.prev, r, "f")
                elif op.kind == BWD and op.next >= 0:
                    need = (op.next, r, "b")
                if need is not None:
                    q = queues.get(need, [])
                    if not q or q[0] != op.mb:
                        break
                    q.pop(0)
                if op.kind == FWD and op.next >= 0:
                    queues.setdefault((r, op.next, "f"), []).append(op.mb)
                if op.kind in (BWD, FWD_BWD) and op.prev >= 0 and not forward_only:
                    queues.setdefault((r, op.prev, "b"), []).append(op.mb)
                pos[r] += 1
                progressed = True
    stuck = {r: ops[pos[r]] for r, ops in plans.items() if pos[r] < len(ops)}
    if stuck:
        r, op = next(iter(stuck.items()))
        raise PlanError(f"deadlock: {len(stuck)} ranks cannot go on, e.g. rank {r} waits at {op}")
