"""Pipeline point-to-point engine, inference ring and metric reduction.

The reference moves every activation through host memory with four Python
threads per rank, blocking gloo send/recv and receive-from-any
(src/comm.py:16-115), and doubles each message with a metadata plane
(src/serializer.py:9-15).  Here:

* sources and destinations come from the static plan (parallel/schedule.py),
  so every receive names its source and no metadata travels;
* transfers are ``isend``/``irecv`` on the device (NCCL over NVLink on GPUs,
  gloo on CPU) in per-direction groups; NCCL runs them on its own streams, the
  compute stream only waits for the receive it is about to consume;
* a receive is posted ``prefetch`` operations of the plan before the operation
  that consumes it, so the transfer of the next microbatch overlaps the compute
  of the current one.  Not earlier: a posted NCCL receive is a kernel that spins
  on the device until its sender shows up, and every SM it sits on cannot take a
  block of a persistent GEMM meanwhile; with static tile assignment one blocked
  SM is enough to stretch each GEMM to two waves.  (Receives posted at the start
  of the step for gradients that arrive 30 ms later made the forwards of the
  fill phase 1.6 times slower.)
"""
from __future__ import annotations

import datetime
import time
from collections import deque
from typing import Deque, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .schedule import BWD, FWD, FWD_BWD, Op
from ..utils.metrics import Outputs, aggregate_outputs


class StepTimeout(RuntimeError):
    pass


class PipelineComm:
    def __init__(self, world, shape: Tuple[int, ...], dtype: torch.dtype, device: torch.device,
                 prefetch: int = 2):
        self.world, self.shape, self.dtype, self.device = world, tuple(shape), dtype, device
        self.prefetch = max(0, prefetch)
        self.is_nccl = world.backend == "nccl"
        self.device_async = self.is_nccl      # the host only queues transfers; the device streams complete them
        self._recv_plan: List[Tuple[int, int, object]] = []   # (op index, src, group)
        self._posted: Deque[Tuple[int, torch.Tensor, object]] = deque()
        self._next_post = 0
        self._sends: List[Tuple[object, torch.Tensor]] = []
        self.deadline: Optional[float] = None
        self.tolerant = False        # set with membership tracking: a failed transfer ends the step like a timeout
        self.bytes_sent = 0

    # -- set-up --------------------------------------------------------------
    def warmup(self) -> None:
        """Create every pair channel up front, in one global order.

        NCCL builds a two-rank communicator the first time a pair talks, and
        that is a blocking hand-shake.  Left to first use inside a step, two
        pairs that wait on each other's partner would deadlock; walking all
        (boundary, direction, sender, receiver) tuples in lexicographic order
        on every rank cannot."""
        w = self.world
        if w.num_stages == 1:
            return
        t = torch.zeros(1, dtype=self.dtype, device=self.device)
        for b in range(w.num_stages - 1):
            for direction in (0, 1):
                grp = w.fwd_groups[b] if direction == 0 else w.bwd_groups[b]
                lo, hi = w.stage2ranks[b], w.stage2ranks[b + 1]
                senders, receivers = (lo, hi) if direction == 0 else (hi, lo)
                for s in senders:
                    for r in receivers:
                        if w.rank == s:
                            dist.send(t, dst=r, group=grp)
                        elif w.rank == r:
                            dist.recv(t, src=s, group=grp)
        if self.is_nccl:
            torch.cuda.synchronize(self.device)

    # -- per step --------------------------------------------------------------
    def begin_step(self, ops: Sequence[Op], timeout_s: Optional[float] = None) -> None:
        w = self.world
        self._recv_plan = []
        for i, op in enumerate(ops):
            if op.kind in (FWD, FWD_BWD) and op.prev >= 0:
                self._recv_plan.append((i, op.prev, w.fwd_groups[w.stage - 1]))
            elif op.kind == BWD and op.next >= 0:
                self._recv_plan.append((i, op.next, w.bwd_groups[w.stage]))
        self._posted.clear()
        self._next_post = 0
        self._sends = []
        self.deadline = time.time() + timeout_s if timeout_s else None
        self.tick(0)

    def tick(self, op_index: int) -> None:
        """The rank is about to run operation ``op_index`` of its plan: post the receives of the operations
        up to ``prefetch`` ahead of it (in plan order, which is the order the peers send in)."""
        while self._next_post < len(self._recv_plan) and self._recv_plan[self._next_post][0] <= op_index + self.prefetch:
            i, src, grp = self._recv_plan[self._next_post]
            buf = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            work = dist.irecv(buf, src=src, group=grp)
            self._posted.append((i, buf, work))
            self._next_post += 1

    def recv(self, op_index: int) -> torch.Tensor:
        """Tensor received for op ``op_index`` (ops must be consumed in plan order)."""
        self.tick(op_index)
        i, buf, work = self._posted.popleft()
        assert i == op_index, f"receive order broken: expected op {i}, asked {op_index}"
        self._wait(work)
        return buf

    def _wait(self, work) -> None:
        if self.is_nccl:
            work.wait()          # stream-level dependency, does not block the host
            return
        if self.deadline is None:
            work.wait()
            return
        remaining = self.deadline - time.time()
        if remaining <= 0:
            raise StepTimeout("pipeline transfer timed out")
        try:
            work.wait(timeout=datetime.timedelta(seconds=remaining))
        except RuntimeError as e:
            # with membership tracking a transfer that fails because its peer is gone ends the step
            # the same way a timeout does
            if self.tolerant or "imeout" in str(e) or "timed out" in str(e):
                raise StepTimeout(str(e)) from e
            raise

    def send_forward(self, tensor: torch.Tensor, dst: int) -> None:
        self._send(tensor, dst, self.world.fwd_groups[self.world.stage])

    def send_backward(self, tensor: torch.Tensor, dst: int) -> None:
        self._send(tensor, dst, self.world.bwd_groups[self.world.stage - 1])

    def _send(self, tensor: torch.Tensor, dst: int, grp) -> None:
        t = tensor.detach()
        if t.dtype != self.dtype:
            t = t.to(self.dtype)
        t = t.contiguous()
        work = dist.isend(t, dst=dst, group=grp)
        self._sends.append((work, t))
        self.bytes_sent += t.numel() * t.element_size()

    def end_step(self) -> None:
        for work, _ in self._sends:
            self._wait(work)
        self._sends = []
        assert not self._posted, "step ended with receives still posted"

    def abandon_step(self) -> None:
        """Forget a step that timed out (reference: break out of the loop with
        a warning, src/train.py:186)."""
        self._posted.clear()
        self._sends = []


class InferenceComm:
    """Ring over stage leaders for sampling (reference: src/comm.py:151-183):
    activations go leader to leader, the last leader returns token ids to the first."""

    def __init__(self, world, device: torch.device):
        self.world, self.device = world, device

    def send_hidden(self, x: torch.Tensor) -> None:
        dist.send(x.contiguous(), dst=self.world.next_stage_leader)

    def recv_hidden(self, shape, dtype) -> torch.Tensor:
        buf = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(buf, src=self.world.prev_stage_leader)
        return buf

    def send_ids(self, ids: torch.Tensor) -> None:
        dist.send(ids.contiguous(), dst=self.world.first_stage_leader)

    def recv_ids(self, shape) -> torch.Tensor:
        buf = torch.empty(shape, dtype=torch.long, device=self.device)
        dist.recv(buf, src=self.world.last_stage_leader)
        return buf


def sync_outputs(world, local: Outputs, device: torch.device) -> Outputs:
    """Stage-wide aggregate of the step outputs.  One all-gather of a packed
    float64 vector replaces the reference's pickled ``all_gather_object``
    (src/comm.py:125-149); the aggregation rule is unchanged."""
    R = world.num_replicas
    if R == 1:
        return local
    v = torch.tensor(local.to_vector(), dtype=torch.float64, device=device)
    out = [torch.empty_like(v) for _ in range(R)]
    dist.all_gather(out, v, group=world.curr_stage_group)
    return aggregate_outputs(local, [Outputs.from_vector(o.tolist()) for o in out])
