"""The stage rendezvous that precedes a fused collective, on two gloo ranks.

Replicas of a one-stage DiLoCo world share nothing for H steps, so they reach an
outer sync with whatever skew has built up; the fused kernel's wait for its
peers is bounded (a dead peer must not hang the GPU), so the skew has to be
absorbed before the kernel is queued.  Here one rank arrives a second late: both
must leave the meeting together, and later than the late rank's arrival.
"""
import os
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank: int, path: str, out):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=2)
    from diloco_swarm_b200.parallel.collectives import StageRendezvous
    group = dist.new_group([0, 1])
    r = StageRendezvous(group, torch.device("cpu"))
    r.meet()                       # first use builds the group's connections
    dist.barrier()
    t0 = time.time()
    if rank == 1:
        time.sleep(1.0)            # the skew
    arrived = time.time() - t0
    r.meet()
    left = time.time() - t0
    out.put((rank, arrived, left, r.count))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.slow
def test_both_replicas_leave_after_the_late_one_arrives():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "store")
        procs = [ctx.Process(target=_worker, args=(r, path, out)) for r in range(2)]
        for p in procs:
            p.start()
        got = sorted(out.get(timeout=120) for _ in range(2))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    (_, a0, l0, c0), (_, a1, l1, c1) = got
    assert a0 < 0.2 and a1 >= 1.0
    assert l0 >= 0.95 and l1 >= 1.0, "the early replica left before the late one had arrived"
    assert abs(l0 - l1) < 0.5
    assert c0 == c1 == 2
