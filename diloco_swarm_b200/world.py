"""S stages x R replicas topology and its process groups.

Same rank arithmetic as the reference (src/world.py:22-29,96-100): stage of a
rank is ``rank % num_stages``, a stage's leader is its lowest rank, the master
is the leader of the last stage.  Differences, all on purpose:

* backend is NCCL on CUDA devices (one process per GPU) and gloo on CPU; the
  reference always uses gloo with CPU staging (src/world.py:33, src/comm.py:38);
* there is no TCP-store step protocol (src/world.py:73-94): the routing table
  is a pure function of (seed, step), see parallel/schedule.py;
* every stage boundary has one group per direction, so activation traffic and
  gradient traffic never queue behind each other on the same channel.
"""
from __future__ import annotations

import datetime
import os
from typing import Any, Dict, Iterator, List, Optional

import torch
import torch.distributed as dist


class World:
    def __init__(self, num_stages: int, device_type: str = "cpu", backend: Optional[str] = None,
                 timeout_s: float = 600.0, init: bool = True):
        self.local_rank = int(os.environ.get("LOCAL_RANK", 0))
        self.rank = int(os.environ.get("RANK", 0))
        self.local_world_size = int(os.environ.get("LOCAL_WORLD_SIZE", 1))
        self.world_size = int(os.environ.get("WORLD_SIZE", 1))
        self.master_addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        self.master_port = int(os.environ.get("MASTER_PORT", 29500))
        self.num_stages = num_stages
        if self.world_size < num_stages:
            raise ValueError("world size must be at least the number of stages")

        self.ranks2stage: Dict[int, int] = {r: r % num_stages for r in range(self.world_size)}
        self.stage2ranks: Dict[int, List[int]] = {
            s: [r for r in range(self.world_size) if r % num_stages == s] for s in range(num_stages)}
        self.stage2leader: Dict[int, int] = {s: self.stage2ranks[s][0] for s in range(num_stages)}
        self.stage = self.ranks2stage[self.rank]
        self.is_first_stage = self.stage == 0
        self.is_last_stage = self.stage == num_stages - 1
        self.is_leader = self.rank == self.stage2leader[self.stage]
        self.is_master = self.is_leader and self.is_last_stage
        self.replica_index = self.stage2ranks[self.stage].index(self.rank)
        self.num_replicas = len(self.stage2ranks[self.stage])

        self.device_type = device_type
        self.backend = backend or ("nccl" if device_type == "cuda" else "gloo")
        self.fwd_groups: Dict[int, Any] = {}   # boundary b (stage b -> b+1) -> group
        self.bwd_groups: Dict[int, Any] = {}
        self.curr_stage_group = None
        self.first_last_stage_group = None
        self._owns_pg = False
        if init:
            self._init_groups(timeout_s)

    # ------------------------------------------------------------------
    def _init_groups(self, timeout_s: float) -> None:
        timeout = datetime.timedelta(seconds=timeout_s)
        if not dist.is_initialized():
            kwargs: Dict[str, Any] = {}
            # Binding the device up front makes NCCL create the communicators eagerly, and
            # then send/recv of a sub-group run on that group's one stream.  Left lazy,
            # every rank pair gets its own point-to-point communicator and stream, which
            # is what the pipeline transport wants.
            if self.backend == "nccl" and os.environ.get("DSWARM_NCCL_EAGER", "0") == "1":
                kwargs["device_id"] = torch.device("cuda", self.local_rank)
            dist.init_process_group(
                backend=self.backend, rank=self.rank, world_size=self.world_size,
                init_method=f"tcp://{self.master_addr}:{self.master_port}", timeout=timeout, **kwargs)
            self._owns_pg = True
        S = self.num_stages
        # all ranks create all groups in the same order
        for b in range(S - 1):
            members = self.stage2ranks[b] + self.stage2ranks[b + 1]
            self.fwd_groups[b] = dist.new_group(members, timeout=timeout)
            self.bwd_groups[b] = dist.new_group(members, timeout=timeout)
        for s in range(S):
            g = dist.new_group(self.stage2ranks[s], timeout=timeout)
            if s == self.stage:
                self.curr_stage_group = g
        fl = sorted(set(self.stage2ranks[0] + self.stage2ranks[S - 1]))
        self.first_last_stage_group = dist.new_group(fl, timeout=timeout)
        self.barrier()

    def regroup(self, alive: List[bool], rebuild_p2p: bool = False) -> None:
        """Shrink this rank's view of the world to the live ranks: stage membership, leaders and the
        stage group used by the collectives (created among the live members only).  Point-to-point
        groups are left alone after a clean leave: transfers only ever involve two live ranks.
        After a step that failed half-way, ``rebuild_p2p`` also replaces the pipeline groups, so that
        receives still posted for the abandoned step can never match a later send.  Every live rank
        must make the same call."""
        S = self.num_stages
        self.stage2ranks = {s: [r for r in range(self.world_size) if r % S == s and alive[r]] for s in range(S)}
        for s in range(S):
            if not self.stage2ranks[s]:
                raise RuntimeError(f"stage {s} has no live replica left")
        self.stage2leader = {s: self.stage2ranks[s][0] for s in range(S)}
        self.is_leader = self.rank == self.stage2leader[self.stage]
        self.is_master = self.is_leader and self.is_last_stage
        mine = self.stage2ranks[self.stage]
        self.num_replicas = len(mine)
        self.replica_index = mine.index(self.rank)
        # Member-only group creation keys its rendezvous on how many groups the process has made so far,
        # so every live rank makes the same calls in the same order, with one-rank groups as fillers
        # where it is not a member (two live ranks whose counts differ would wait for each other forever).
        g = dist.new_group(mine, use_local_synchronization=True)
        self.curr_stage_group = g if len(mine) > 1 else None
        if rebuild_p2p:
            for b in range(S - 1):                 # ascending on every rank: the rendezvous chain starts at boundary 0
                members = self.stage2ranks[b] + self.stage2ranks[b + 1]
                if self.rank in members:
                    self.fwd_groups[b] = dist.new_group(members, use_local_synchronization=True)
                    self.bwd_groups[b] = dist.new_group(members, use_local_synchronization=True)
                else:
                    dist.new_group([self.rank], use_local_synchronization=True)
                    dist.new_group([self.rank], use_local_synchronization=True)

    def barrier(self) -> None:
        if dist.is_initialized():
            if self.backend == "nccl":
                dist.barrier(device_ids=[self.local_rank])
            else:
                dist.barrier()

    def destroy(self) -> None:
        if dist.is_initialized() and self._owns_pg:
            dist.destroy_process_group()

    # ------------------------------------------------------------------
    @property
    def has_next_stage(self) -> bool:
        return self.stage + 1 < self.num_stages

    @property
    def has_prev_stage(self) -> bool:
        return self.stage > 0

    @property
    def next_stage_leader(self) -> int:
        return self.stage2leader[self.stage + 1]

    @property
    def prev_stage_leader(self) -> int:
        return self.stage2leader[self.stage - 1]

    @property
    def first_stage_leader(self) -> int:
        return self.stage2leader[0]

    @property
    def last_stage_leader(self) -> int:
        return self.stage2leader[self.num_stages - 1]

    @property
    def first_stage_ranks(self) -> List[int]:
        return self.stage2ranks[0]

    @property
    def last_stage_ranks(self) -> List[int]:
        return self.stage2ranks[self.num_stages - 1]

    @property
    def stage_ranks(self) -> List[int]:
        return self.stage2ranks[self.stage]

    def __repr__(self) -> str:
        return (f"World(rank={self.rank}, stage={self.stage}, is_first_stage={self.is_first_stage}, "
                f"is_last_stage={self.is_last_stage}, is_master={self.is_master}, is_leader={self.is_leader})")

    def as_dict(self) -> Dict[str, Any]:
        return {"local_rank": self.local_rank, "rank": self.rank,
                "local_world_size": self.local_world_size, "world_size": self.world_size,
                "master_addr": self.master_addr, "master_port": self.master_port,
                "num_stages": self.num_stages, "is_master": self.is_master, "is_leader": self.is_leader}

    def __iter__(self) -> Iterator:
        return iter(self.as_dict().items())
