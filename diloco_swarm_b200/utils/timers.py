"""Device-side phase timers.

The reference times a step with ``time.time()`` around everything
(src/train.py:162,272).  Here each phase of a step (pipeline work, gradient
sync, optimiser, outer sync) is bracketed by CUDA events on the compute stream,
so the times are device times and recording them costs no synchronisation;
they are read after the step's one host sync.  On CPU the timer falls back to
wall-clock time.  ``nvtx=True`` also opens an NVTX range per phase for
timeline tools.
"""
from __future__ import annotations

import time
from contextlib import contextmanager
from typing import Dict, List, Tuple

import torch


class PhaseTimer:
    def __init__(self, device: torch.device, nvtx: bool = False):
        self.cuda = device.type == "cuda"
        self.nvtx = nvtx and self.cuda
        self._pending: List[Tuple[str, object, object]] = []
        self._wall: Dict[str, float] = {}

    @contextmanager
    def phase(self, name: str):
        if self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if self.nvtx:
                torch.cuda.nvtx.range_push(name)
            e0.record()
            try:
                yield
            finally:
                e1.record()
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
                self._pending.append((name, e0, e1))
        else:
            t0 = time.time()
            try:
                yield
            finally:
                self._wall[name] = self._wall.get(name, 0.0) + (time.time() - t0) * 1e3

    def collect(self) -> Dict[str, float]:
        """Milliseconds per phase since the last call.  Call after a device synchronize."""
        out = dict(self._wall)
        for name, e0, e1 in self._pending:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        self._pending, self._wall = [], {}
        return out
