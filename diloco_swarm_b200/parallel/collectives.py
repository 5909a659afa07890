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


class StageRendezvous:
    """Brings the replicas of a stage together, on the device, before a fused collective is queued.

    The fused kernels bound their waits for a peer (``swarm.peer_wait_s``), which is right for telling a
    dead peer from a live one but wrong for absorbing skew: DiLoCo replicas of a one-stage world share
    nothing for H steps, and a few per cent of clock difference under the power cap adds up to seconds.
    (The reference meets at a ``dist.barrier()`` every step, src/train.py:246.)  One tiny all-reduce on the
    stage group, queued on the stream the fused kernel will run on, makes every replica's stream wait
    until all have arrived; the kernel's own bounded wait then only sees the microseconds between the
    replicas leaving that all-reduce."""

    def __init__(self, group, device: torch.device):
        self.group, self.device = group, device
        self.token = torch.zeros(1, dtype=torch.float32, device=device)
        self.count = 0

    def meet(self, stream: Optional["torch.cuda.Stream"] = None) -> None:
        if self.group is None or dist.get_world_size(self.group) == 1:
            return
        self.count += 1
        if stream is not None and self.device.type == "cuda":
            with torch.cuda.stream(stream):
                dist.all_reduce(self.token, group=self.group)
        else:
            dist.all_reduce(self.token, group=self.group)


def wait_cycles_for(seconds: float) -> int:
    """Cycle budget of a peer wait (the kernels read clock64; 2 GHz nominal)."""
    return max(1, int(seconds * 2.0e9))


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
        if self.R > 1 and self.theta.mc_ptr:
            # the weights are bound to a multicast object: reduce and broadcast inside the NVSwitch
            check(cuda_lib().dsw_outer_sync_nvls(
                self.theta.table, self.theta.mc_ptr, self.flags.table, self.theta_g.data_ptr(), self.mom.data_ptr(),
                self.n, self.shard, self.rank, self.R, self.lr, self.mu, 1 if self.nesterov else 0, self.seq,
                self.wait_cycles, self.blocks, self.status.ptr if self.status else None, stream_ptr()),
                "dsw_outer_sync_nvls")
            self.seq += 2
            return
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
        self.nvls = bool(grad.mc_ptr)
        self.stage_buf = SymmetricBuffer(n * 2, device, group, multicast=self.nvls) if (wire_bf16 and self.R > 1) else None
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
        if self.nvls:
            mc = self.stage_buf.mc_ptr if self.wire_bf16 else self.grad.mc_ptr
            check(cuda_lib().dsw_grad_allreduce_nvls(
                table, mc, self.flags.table, self.grad.ptr, offset, count, shard, self.rank, self.R,
                1 if self.wire_bf16 else 0, self.seq, self.wait_cycles, self.blocks,
                self.status.ptr if self.status else None, stream_ptr(stream)), "dsw_grad_allreduce_nvls")
            self.seq += 2
            return
        check(cuda_lib().dsw_grad_allreduce(
            table, self.flags.table, self.grad.ptr, offset, count, shard, self.rank, self.R,
            1 if self.wire_bf16 else 0, self.seq, self.wait_cycles, 1, 7, self.blocks,
            self.status.ptr if self.status else None, stream_ptr(stream)), "dsw_grad_allreduce")
        self.seq += 2

    def all(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        self.bucket(0, self.n, stream)


def check_against_nccl(group, device: torch.device, n: int, buckets, lr: float = 0.7, momentum: float = 0.9,
                       seed: int = 1234, multicast: bool = False) -> dict:
    """Run the fused collectives once on fresh buffers of a stage's real size and bucket list and compare
    them with the library route (NCCL all-reduce + separate update) on the same values.

    Returns ``{"status": "ok" | "mismatch" | "n/a", ...}`` with the largest absolute differences; every rank
    of ``group`` must call it (it allocates symmetric buffers collectively).  Meant for places where the
    multi-GPU path has to prove itself on the box it runs on, e.g. the benchmark outside its timed regions."""
    R = dist.get_world_size(group) if group is not None else 1
    if R == 1:
        return {"status": "n/a", "why": "one replica per stage: no stage-wide collective runs"}
    rank = dist.get_rank(group)
    status = Status(device)
    g = torch.Generator(device=device).manual_seed(seed + rank)
    out = {"status": "ok", "replicas": R, "elements": n, "buckets": len(buckets), "nvls": False}

    def worst(x: torch.Tensor) -> float:
        t = x.abs().max().reshape(1).to(torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t.item())

    # ---- per-step gradient all-reduce, fp32 and bf16 wire, bucket by bucket as the engine sends them
    for wire in (False, True):
        buf = SymmetricBuffer(n * 4, device, group, multicast=multicast)
        out["nvls"] = bool(buf.mc_ptr)
        grad = buf.view(torch.float32, n)
        grad.copy_(torch.randn(n, device=device, generator=g) * 1e-2)
        ref = grad.clone()
        dist.all_reduce(ref, group=group)
        ref.div_(R)
        gs = GradSync(buf, n, device, group, wire_bf16=wire, status=status)
        torch.cuda.synchronize(device)
        dist.barrier(group=group, device_ids=[device.index])
        for off, cnt in buckets:
            gs.bucket(off, cnt)
        torch.cuda.synchronize(device)
        err = worst(grad - ref)
        tol = 5e-4 if wire else 1e-6        # bf16 wire: two roundings of values up to about 6e-2
        out["grad_allreduce_bf16_wire_max_err" if wire else "grad_allreduce_f32_max_err"] = err
        if not err <= tol:
            out["status"] = "mismatch"
        dist.barrier(group=group, device_ids=[device.index])
    # ---- DiLoCo outer sync
    theta_buf = SymmetricBuffer(n * 4, device, group, multicast=multicast)
    theta = theta_buf.view(torch.float32, n)
    common = torch.Generator(device=device).manual_seed(seed)
    theta_g = torch.randn(n, device=device, generator=common)
    theta.copy_(theta_g)                                   # OuterSync takes its shard of the global weights from here
    sync = OuterSync(theta_buf, n, device, lr, momentum, True, group, status)
    theta.add_(torch.randn(n, device=device, generator=g) * 1e-2)       # H inner steps' worth of drift, per replica
    delta = theta_g - theta
    dist.all_reduce(delta, group=group)
    delta.div_(R)
    ref = theta_g - lr * (delta + momentum * delta)        # first Nesterov step: buffer = delta
    torch.cuda.synchronize(device)
    dist.barrier(group=group, device_ids=[device.index])
    sync.step()
    torch.cuda.synchronize(device)
    err = worst(theta - ref)
    out["outer_sync_max_err"] = err
    if not err <= 1e-5:
        out["status"] = "mismatch"
    code = status.read()
    if code != 0:
        out["status"], out["kernel_status"] = "mismatch", code
    dist.barrier(group=group, device_ids=[device.index])
    return out
