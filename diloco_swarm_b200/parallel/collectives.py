"""Host side of the fused stage-wide synchronisations (csrc/collectives.cu).

``OuterSync``  DiLoCo outer step: all-reduce of (theta_global - theta_local)
               over the stage's replicas + Nesterov momentum + write-back, one
               kernel (reference: src/train.py:261-269).
``GradSync``   per-step gradient averaging of plain SWARM, one kernel per
               bucket, fp32 or bf16 on the wire (reference: src/comm.py:117-123).

Both have a library twin (``collective="nccl"``): NCCL all-reduce followed by
separate update kernels, which is the baseline the fused kernels are measured
against.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops._lib import Status, check, cuda_lib, stream_ptr
from .symm import FLAG_WORDS, SymmetricBuffer


def touch_map(offset: int, count: int, shard: int, R: int, rank: int, phase: int, grid: int, block: int,
              vec: int = 8):
    """Which block of the bf16-wire gradient all-reduce touches which vector of a bucket in a phase
    (0 cast-in, 1 reduce, 2 widen-out) on replica ``rank``; -1 where the phase touches nothing.
    Evaluated by the host library from the same header the kernel walks its indices with
    (csrc/coll_index.h), so a CPU test can check what the per-block barrier relies on."""
    import ctypes

    import numpy as np

    from .schedule import _host
    out = np.empty(count // vec, dtype=np.int32)
    rc = _host().dsw_coll_touch_map(offset, count, shard, R, rank, phase, grid, block, vec,
                                    out.ctypes.data_as(ctypes.c_void_p))
    if rc != 0:
        raise ValueError("bad arguments for the touch map")
    return out


def shard_size(n: int, R: int, align: int) -> int:
    per = (n + R - 1) // R
    return (per + align - 1) // align * align


class OuterSync:
    def __init__(self, theta: SymmetricBuffer, n: int, device: torch.device, lr: float, momentum: float,
                 nesterov: bool, group=None, status: Optional[Status] = None, wait_cycles: int = 0,
                 blocks: int = 0):
        assert n % 4 == 0
        self.theta, self.n, self.device, self.group = theta, n, device, group
        self.R, self.rank = theta.R, theta.rank_in_group
        self.lr, self.mu, self.nesterov = lr, momentum, nesterov
        self.shard = shard_size(n, self.R, 4)
        lo = self.rank * self.shard
        self.lo, self.hi = lo, min(n, lo + self.shard)
        # this replica's 1/R of the global weights and of the momentum
        self.theta_g = theta.view(torch.float32, n)[self.lo:self.hi].clone()
        if self.theta_g.numel() < self.shard:
            self.theta_g = torch.cat([self.theta_g, torch.zeros(self.shard - self.theta_g.numel(), device=device)])
        self.mom = torch.zeros(self.shard, dtype=torch.float32, device=device)
        self.flags = SymmetricBuffer(FLAG_WORDS * 4, device, group) if self.R > 1 else None
        self.seq = 1
        self.status = status
        self.wait_cycles = wait_cycles
        self.blocks = blocks
        if self.R > 1:
            dist.barrier(group=group, device_ids=[device.index])

    def step(self) -> None:
        check(cuda_lib().dsw_outer_sync(
            self.theta.table, self.flags.table if self.flags else None, self.theta_g.data_ptr(), self.mom.data_ptr(),
            self.n, self.shard, self.rank, self.R, self.lr, self.mu, 1 if self.nesterov else 0, self.seq,
            self.wait_cycles, 1 if self.R > 1 else 0, self.blocks, self.status.ptr if self.status else None,
            stream_ptr()), "dsw_outer_sync")
        self.seq += 2

    # checkpoint: every replica contributes its shard; the gathered tensors are
    # the full global weights and momentum of the stage.
    def gather_state(self):
        if self.R == 1:
            return {"theta_g": self.theta_g[:self.n].cpu(), "momentum": self.mom[:self.n].cpu()}
        tg = [torch.empty_like(self.theta_g) for _ in range(self.R)]
        mo = [torch.empty_like(self.mom) for _ in range(self.R)]
        dist.all_gather(tg, self.theta_g, group=self.group)
        dist.all_gather(mo, self.mom, group=self.group)
        return {"theta_g": torch.cat(tg)[:self.n].cpu(), "momentum": torch.cat(mo)[:self.n].cpu()}

    def reset(self) -> None:
        """This replica's shard of the global weights := the same slice of its current weights; momentum := 0."""
        k = self.hi - self.lo
        self.theta_g.zero_()
        self.theta_g[:k].copy_(self.theta.view(torch.float32, self.n)[self.lo:self.hi])
        self.mom.zero_()

    def load_state(self, st) -> None:
        full_t = torch.zeros(self.shard * self.R)
        full_m = torch.zeros(self.shard * self.R)
        full_t[:self.n] = st["theta_g"]
        full_m[:self.n] = st["momentum"]
        self.theta_g.copy_(full_t[self.rank * self.shard:(self.rank + 1) * self.shard])
        self.mom.copy_(full_m[self.rank * self.shard:(self.rank + 1) * self.shard])


class GradSync:
    def __init__(self, grad: SymmetricBuffer, n: int, device: torch.device, group=None, wire_bf16: bool = False,
                 status: Optional[Status] = None, wait_cycles: int = 0, blocks: int = 0):
        assert n % 8 == 0
        self.grad, self.n, self.device, self.group = grad, n, device, group
        self.R, self.rank = grad.R, grad.rank_in_group
        self.wire_bf16 = wire_bf16
        self.stage_buf = SymmetricBuffer(n * 2, device, group) if (wire_bf16 and self.R > 1) else None
        self.flags = SymmetricBuffer(FLAG_WORDS * 4, device, group) if self.R > 1 else None
        self.seq = 1
        self.status = status
        self.wait_cycles = wait_cycles
        self.blocks = blocks
        if self.R > 1:
            dist.barrier(group=group, device_ids=[device.index])

    def bucket(self, offset: int, count: int, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Average elements [offset, offset+count) of the flat gradient over the replicas."""
        if self.R == 1:
            return
        assert offset % 8 == 0 and count % 8 == 0
        shard = shard_size(count, self.R, 8)
        table = self.stage_buf.table if self.wire_bf16 else self.grad.table
        check(cuda_lib().dsw_grad_allreduce(
            table, self.flags.table, self.grad.ptr, offset, count, shard, self.rank, self.R,
            1 if self.wire_bf16 else 0, self.seq, self.wait_cycles, 1, 7, self.blocks,
            self.status.ptr if self.status else None, stream_ptr(stream)), "dsw_grad_allreduce")
        self.seq += 2

    def all(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        self.bucket(0, self.n, stream)
