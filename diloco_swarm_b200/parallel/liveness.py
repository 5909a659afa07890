"""Host-side membership: who takes part in the next step.

The reference has a static world: a rank that dies hangs gloo, and the only
guard is a per-step wall-clock timeout (src/train.py:186).  SWARM's premise is
that any replica of a stage can serve any microbatch, so here the set of live
ranks is an input of the routing function (parallel/schedule.py: ``alive``) and
this module maintains it on the host, between steps, over a TCP store:

* every rank reports ``done/<step>/<rank>`` when it has finished a step;
* a rank that is about to leave writes ``left/<rank>`` = the last step it takes
  part in, then finishes that step and exits cleanly;
* before step t the coordinator (rank 0) waits, up to ``timeout_s``, for the
  ``done`` marks of step t-1 from every rank it believed alive, drops the ranks
  that announced a leave or did not report, and publishes ``alive/<t>``; all
  other ranks wait for that key.  Everybody therefore routes step t with the
  same mask, and nobody launches work for a rank that is gone;
* a rank that dies without a word is noticed inside a step: transfers with it
  fail or time out.  After its pipeline work every rank votes ``ok/<step>/<rank>``;
  the coordinator publishes one verdict per step (all present and all fine, or
  not), so either every live rank applies the step's gradients or none does, and
  the ranks that did not vote are dropped before the next step.

Failures are only ever injected on the host (a rank that leaves, a rank that
stops reporting); nothing here touches a device.  The coordinator itself is
assumed to stay.
"""
from __future__ import annotations

import datetime
import time
from typing import List

import torch.distributed as dist


class Membership:
    def __init__(self, rank: int, world_size: int, host: str, port: int, timeout_s: float = 30.0):
        self.rank, self.world_size, self.timeout_s = rank, world_size, timeout_s
        self.store = dist.TCPStore(host_name=host, port=port, world_size=world_size, is_master=(rank == 0),
                                   timeout=datetime.timedelta(seconds=max(60.0, 4 * timeout_s)),
                                   wait_for_workers=True)
        self.alive: List[bool] = [True] * world_size
        self._silent: set = set()          # coordinator: ranks that missed a vote

    # -- participants -------------------------------------------------------
    def announce_leave(self, last_step: int) -> None:
        """This rank takes part in steps up to ``last_step`` and then exits."""
        self.store.set(f"left/{self.rank}", str(last_step))

    def end_step(self, step: int) -> None:
        self.store.set(f"done/{step}/{self.rank}", "1")

    def begin_step(self, step: int) -> List[bool]:
        """Mask of the ranks that take part in ``step`` (same on every rank)."""
        if self.rank == 0:
            self._publish(step)
        key = f"alive/{step}"
        self.store.wait([key], datetime.timedelta(seconds=4 * self.timeout_s + 30))
        mask = self.store.get(key).decode()
        self.alive = [c == "1" for c in mask]
        return list(self.alive)

    def vote(self, step: int, ok: bool, wait_s: float) -> bool:
        """Common verdict on ``step``: True when every live rank reports that its part of the step went
        through.  ``wait_s`` bounds how long the coordinator waits for the votes (a rank may still be
        inside its step's own timeout)."""
        self.store.set(f"ok/{step}/{self.rank}", "1" if ok else "0")
        if self.rank == 0:
            deadline = time.time() + wait_s
            pending = [r for r in range(self.world_size) if self.alive[r]]
            while pending and time.time() < deadline:
                pending = [r for r in pending if not self.store.check([f"ok/{step}/{r}"])]
                if pending:
                    time.sleep(0.01)
            self._silent.update(pending)
            fine = not pending and all(self.store.get(f"ok/{step}/{r}") == b"1"
                                       for r in range(self.world_size) if self.alive[r])
            self.store.set(f"verdict/{step}", "1" if fine else "0")
        key = f"verdict/{step}"
        self.store.wait([key], datetime.timedelta(seconds=wait_s + 4 * self.timeout_s + 30))
        return self.store.get(key) == b"1"

    # -- coordinator ----------------------------------------------------------
    def _publish(self, step: int) -> None:
        alive = list(self.alive)
        for r in self._silent:                     # missed a vote: gone, no need to wait for its report
            alive[r] = False
        self._silent = set()
        if step > 1:
            deadline = time.time() + self.timeout_s
            pending = [r for r in range(self.world_size) if alive[r] and r != 0]
            while pending and time.time() < deadline:
                pending = [r for r in pending if not self.store.check([f"done/{step - 1}/{r}"])]
                if pending:
                    time.sleep(0.01)
            for r in pending:                      # stopped reporting: treated as gone
                alive[r] = False
        for r in range(self.world_size):
            if alive[r] and self.store.check([f"left/{r}"]):
                if int(self.store.get(f"left/{r}").decode()) < step:
                    alive[r] = False
        self.alive = alive
        self.store.set(f"alive/{step}", "".join("1" if a else "0" for a in alive))
        self._forget(step - 3)

    def _forget(self, step: int) -> None:
        """Drop the keys of a step that every rank has long left, so a long run does not grow the store."""
        if step < 1:
            return
        for key in [f"alive/{step}", f"verdict/{step}"] + [f"{kind}/{step}/{r}" for kind in ("done", "ok")
                                                            for r in range(self.world_size)]:
            try:
                self.store.delete_key(key)
            except Exception:          # a key that was never written
                pass

    def barrier(self, name: str) -> None:
        """Barrier over the ranks currently alive (the process-group barrier would wait for the dead)."""
        n = sum(self.alive)
        self.store.add(f"bar/{name}", 1)
        deadline = time.time() + 4 * self.timeout_s + 30
        while int(self.store.add(f"bar/{name}", 0)) < n:
            if time.time() > deadline:
                raise TimeoutError(f"membership barrier {name!r} timed out")
            time.sleep(0.01)
