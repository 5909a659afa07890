"""Seeded routing table and static per-rank plan (bindings of csrc/schedule.cpp).

Replaces three things in the reference at once: the sender-side
``random.choice`` (src/comm.py:91), receive-from-any-source (src/comm.py:67)
and the TCP-store step counter (src/world.py:73-94).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

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
