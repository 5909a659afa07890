"""A small discrete-event model of warp-specialised kernels: roles, mbarriers, an in-order tensor pipe
and asynchronous copies, with hazard checks on the buffers they share.

The kernels of ``csrc/attention.cu`` and ``csrc/gemm_kernels.cuh`` are sets of single-purpose roles (a TMA
producer, an MMA issuer, row or epilogue warps, a reducer) that hand buffers to one another through
mbarriers.  A wrong parity, a missing wait or a barrier that nobody arrives at does not show as a wrong
number on the GPU; it shows as a wait that runs out, or as a race that the next timing change uncovers.
This module replays such a protocol on the CPU with randomised latencies and checks two things that a
run on the GPU does not: every role runs to its end (no deadlock), and no buffer is written while an
earlier reader or writer of it is still outstanding (no hazard).  The reference has no counterpart (it
ships no kernels).

A role is a Python generator that yields requests:

    ("wait", bar, parity)        block until the phase of that parity has completed
    ("arrive", bar)              one arrival
    ("delay", ns)                the role is busy for that long
    ("mma", reads, writes, ns)   queue a product on the in-order tensor pipe (returns at once)
    ("commit", bar)              arrive on ``bar`` when every product queued so far is done
    ("copy", reads, writes, ns, bar_or_None, done_cb)
                                 an asynchronous copy (TMA load / store / reduction): the source is read
                                 and the destination written during [now, now + ns], then ``bar`` gets one
                                 arrival and ``done_cb`` (if any) runs
    ("read", buf) / ("write", buf)    the role itself touches a buffer now (registers <-> memory)

``reads`` / ``writes`` are lists of buffer names.  A write to a buffer while an asynchronous read or write
of it is outstanding, or a read while an asynchronous write is outstanding, is a hazard.  An entry may also
be a pair: ``(buffer, version)``.  A write leaves its version in the buffer when it completes, a read that
names a version must find exactly that one: a producer that overwrites data its consumer has not taken yet,
or a consumer that runs ahead of its producer, is a hazard too even when the two never overlap in time.
"""
from __future__ import annotations

import heapq
import itertools
from typing import Callable, Dict, Generator, List, Optional, Tuple


class Barrier:
    def __init__(self, name: str, count: int):
        self.name, self.count = name, count
        self.pending = count
        self.phase = 0                      # phases completed so far

    def arrive(self) -> None:
        self.pending -= 1
        assert self.pending >= 0, f"{self.name}: more arrivals than its count"
        if self.pending == 0:
            self.pending = self.count
            self.phase += 1

    def done(self, parity: int) -> bool:
        """mbarrier.try_wait.parity: true once the phase with that parity has completed, i.e. the phase in
        progress has the other parity."""
        return (self.phase & 1) != (parity & 1)


class Hazard(AssertionError):
    pass


class Deadlock(AssertionError):
    pass


class Sim:
    def __init__(self):
        self.now = 0.0
        self._events: List[Tuple[float, int, Callable[[], None]]] = []
        self._seq = itertools.count()
        self.roles: Dict[str, Generator] = {}
        self._blocked: Dict[str, Tuple[Barrier, int]] = {}
        self._finished: Dict[str, bool] = {}
        self.async_reads: Dict[str, int] = {}
        self.async_writes: Dict[str, int] = {}
        self.version: Dict[str, object] = {}
        self._pipe_free_at = 0.0            # the in-order tensor pipe
        self._pipe_pending = 0
        self._commit_waiters: List[Tuple[int, Barrier]] = []
        self._pipe_issued = 0
        self._pipe_done = 0
        self.log: List[str] = []

    # ------------------------------------------------------------------ plumbing
    def at(self, t: float, fn: Callable[[], None]) -> None:
        heapq.heappush(self._events, (t, next(self._seq), fn))

    def add_role(self, name: str, gen: Generator) -> None:
        self.roles[name] = gen
        self._finished[name] = False
        self.at(0.0, lambda: self._step(name))

    @staticmethod
    def _name(entry):
        return entry[0] if isinstance(entry, tuple) else entry

    def _check_version(self, entry, who: str) -> None:
        if isinstance(entry, tuple) and self.version.get(entry[0]) != entry[1]:
            raise Hazard(f"t={self.now:.0f}: {who} reads {entry[0]} expecting version {entry[1]!r}, "
                         f"finds {self.version.get(entry[0])!r}")

    def _begin_async(self, reads, writes) -> None:
        for e in reads:
            self._check_version(e, "an asynchronous operation")
        tagged = [e for e in writes if isinstance(e, tuple)]
        reads, writes = [self._name(e) for e in reads], [self._name(e) for e in writes]
        self._begin_plain(reads, writes)
        return tagged

    def _begin_plain(self, reads, writes) -> None:
        for b in writes:
            if self.async_reads.get(b, 0) or self.async_writes.get(b, 0):
                raise Hazard(f"t={self.now:.0f}: asynchronous write of {b} while it is still being read or written")
        for b in reads:
            if self.async_writes.get(b, 0):
                raise Hazard(f"t={self.now:.0f}: asynchronous read of {b} while it is still being written")
        for b in reads:
            self.async_reads[b] = self.async_reads.get(b, 0) + 1
        for b in writes:
            self.async_writes[b] = self.async_writes.get(b, 0) + 1

    def _end_async(self, reads, writes) -> None:
        for e in reads:
            self.async_reads[self._name(e)] -= 1
        for e in writes:
            self.async_writes[self._name(e)] -= 1
            if isinstance(e, tuple):
                self.version[e[0]] = e[1]

    def _arrive(self, bar: Barrier) -> None:
        bar.arrive()
        for name, (b, parity) in list(self._blocked.items()):
            if b is bar and bar.done(parity):
                del self._blocked[name]
                self.at(self.now, lambda n=name: self._step(n))

    def _pipe_complete(self, reads, writes) -> None:
        self._end_async(reads, writes)
        self._pipe_done += 1
        keep = []
        for upto, bar in self._commit_waiters:
            if self._pipe_done >= upto:
                self._arrive(bar)
            else:
                keep.append((upto, bar))
        self._commit_waiters = keep

    # ------------------------------------------------------------------ one role, until it blocks
    def _step(self, name: str) -> None:
        gen = self.roles[name]
        while True:
            try:
                req = next(gen)
            except StopIteration:
                self._finished[name] = True
                return
            kind = req[0]
            if kind == "wait":
                _, bar, parity = req
                if not bar.done(parity):
                    self._blocked[name] = (bar, parity)
                    return
            elif kind == "arrive":
                self._arrive(req[1])
            elif kind == "delay":
                self.at(self.now + req[1], lambda n=name: self._step(n))
                return
            elif kind == "mma":
                _, reads, writes, ns = req
                # operands are read and the accumulator written while the product runs, after everything
                # queued before it (the pipe is in order)
                start = max(self.now, self._pipe_free_at)
                self._pipe_free_at = start + ns
                self._pipe_issued += 1
                self.at(start, lambda r=reads, w=writes: self._begin_async(r, w))
                self.at(start + ns, lambda r=reads, w=writes: self._pipe_complete(r, w))
            elif kind == "commit":
                if self._pipe_done >= self._pipe_issued:
                    self._arrive(req[1])
                else:
                    self._commit_waiters.append((self._pipe_issued, req[1]))
            elif kind == "copy":
                _, reads, writes, ns, bar, cb = req
                self._begin_async(reads, writes)

                def fin(r=reads, w=writes, b=bar, c=cb):
                    self._end_async(r, w)
                    if b is not None:
                        self._arrive(b)
                    if c is not None:
                        c()
                self.at(self.now + ns, fin)
            elif kind == "read":
                b = self._name(req[1])
                if self.async_writes.get(b, 0):
                    raise Hazard(f"t={self.now:.0f}: {name} reads {b} while it is still being written")
                self._check_version(req[1], name)
            elif kind == "write":
                b = self._name(req[1])
                if self.async_reads.get(b, 0) or self.async_writes.get(b, 0):
                    raise Hazard(f"t={self.now:.0f}: {name} writes {b} while it is still being read or written")
                if isinstance(req[1], tuple):
                    self.version[b] = req[1][1]
            else:
                raise ValueError(kind)

    def run(self, limit_events: int = 2_000_000) -> float:
        n = 0
        while self._events:
            t, _, fn = heapq.heappop(self._events)
            self.now = t
            fn()
            n += 1
            if n > limit_events:
                raise Deadlock("event limit reached")
        stuck = [f"{r} on {b.name} (parity {p}, phase {b.phase})" for r, (b, p) in self._blocked.items()]
        unfinished = [r for r, f in self._finished.items() if not f]
        if unfinished:
            raise Deadlock("roles that never finished: " + "; ".join(stuck or unfinished))
        return self.now
