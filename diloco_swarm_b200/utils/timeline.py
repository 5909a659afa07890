"""Per-operation timeline of training steps, one lane per rank.

The reference times a whole step with ``time.time()`` (src/train.py:162,272) and has no view of
where inside a step a rank computes and where it waits.  With ``--logging.timeline_steps N`` every
rank records the start and end of each forward / backward of N steps (CUDA events on the compute
stream on GPUs, the wall clock on CPU; nothing is synchronised beyond the step's own sync) and
appends them to ``<run>/timeline/<rank>.jsonl`` (on GPUs also when the host queued each of them, which
shows whether the device waits for the host or for a peer).  This module's command line merges the per-rank
files into one trace that chrome://tracing or Perfetto shows as a pipeline diagram, and prints how
busy every rank was:

    python -m diloco_swarm_b200.utils.timeline logs/<run>/timeline --out trace.json

Ranks are aligned by the host clock taken when each rank records the first event of a step; on one
machine that is good to well under a millisecond, which is enough to see pipeline bubbles.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import time
from contextlib import contextmanager
from typing import Dict, List, Optional, Tuple

import torch


class StepTimeline:
    def __init__(self, device: torch.device, out_dir: str, rank: int):
        self.cuda = device.type == "cuda"
        self.path = os.path.join(out_dir, f"{rank}.jsonl")
        os.makedirs(out_dir, exist_ok=True)
        self.rank = rank
        self.step: Optional[int] = None
        self._t0_host = 0.0
        self._t0_event = None
        self._ops: List[Tuple[str, object, object]] = []
        self._host: List[Tuple[str, float, float]] = []

    def begin_step(self, step: int) -> None:
        self.step, self._ops, self._host = step, [], []
        if self.cuda:
            self._t0_event = torch.cuda.Event(enable_timing=True)
            torch.cuda.current_stream().synchronize()      # host clock and device clock meet here
            self._t0_host = time.time()
            self._t0_event.record()
        else:
            self._t0_host = time.time()

    @contextmanager
    def op(self, name: str):
        if self.step is None:
            yield
            return
        if self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            h0 = time.time()
            e0.record()
            try:
                yield
            finally:
                e1.record()
                self._ops.append((name, e0, e1))
                self._host.append((name, h0, time.time()))     # when the host queued the same work
        else:
            t0 = time.time()
            try:
                yield
            finally:
                self._ops.append((name, t0, time.time()))

    def end_step(self) -> None:
        """Write the step's operations.  Call after the step's device synchronize."""
        if self.step is None:
            return
        rows = []
        for name, a, b in self._ops:
            if self.cuda:
                start, end = self._t0_event.elapsed_time(a), self._t0_event.elapsed_time(b)
            else:
                start, end = (a - self._t0_host) * 1e3, (b - self._t0_host) * 1e3
            rows.append({"name": name, "start_ms": start, "end_ms": end})
        host = [{"name": n, "start_ms": (a - self._t0_host) * 1e3, "end_ms": (b - self._t0_host) * 1e3}
                for n, a, b in self._host]
        with open(self.path, "a") as f:
            f.write(json.dumps({"rank": self.rank, "step": self.step, "t0": self._t0_host, "ops": rows,
                                "host": host}) + "\n")
        self.step, self._ops, self._host = None, [], []


# ---------------------------------------------------------------------- merging and reading
def load(timeline_dir: str) -> List[dict]:
    """All recorded (rank, step) records of a run."""
    out = []
    for path in sorted(glob.glob(os.path.join(timeline_dir, "*.jsonl"))):
        with open(path) as f:
            out.extend(json.loads(line) for line in f if line.strip())
    return out


def chrome_trace(records: List[dict]) -> dict:
    """Trace-event JSON (one process per rank, microseconds since the earliest step start)."""
    if not records:
        return {"traceEvents": []}
    origin = min(r["t0"] for r in records)
    events = []
    for r in records:
        base_us = (r["t0"] - origin) * 1e6
        for op in r["ops"]:
            events.append({"name": op["name"], "cat": f"step {r['step']}", "ph": "X", "pid": r["rank"], "tid": 0,
                           "ts": base_us + op["start_ms"] * 1e3, "dur": max(0.0, op["end_ms"] - op["start_ms"]) * 1e3})
        for op in r.get("host", []):        # GPUs only: the host's enqueue of the same operations, on a second lane
            events.append({"name": op["name"], "cat": f"step {r['step']}", "ph": "X", "pid": r["rank"], "tid": 1,
                           "ts": base_us + op["start_ms"] * 1e3, "dur": max(0.0, op["end_ms"] - op["start_ms"]) * 1e3})
    for rank in sorted({r["rank"] for r in records}):
        events.append({"name": "process_name", "ph": "M", "pid": rank, "args": {"name": f"rank {rank}"}})
    return {"traceEvents": events, "displayTimeUnit": "ms"}


def utilisation(records: List[dict]) -> Dict[int, Dict[str, float]]:
    """Per step: the span from the earliest start to the latest end over all ranks, and the share of it
    that every rank spent inside its operations."""
    out: Dict[int, Dict[str, float]] = {}
    for step in sorted({r["step"] for r in records}):
        recs = [r for r in records if r["step"] == step and r["ops"]]
        if not recs:
            continue
        origin = min(r["t0"] for r in recs)
        first = min((r["t0"] - origin) * 1e3 + min(o["start_ms"] for o in r["ops"]) for r in recs)
        last = max((r["t0"] - origin) * 1e3 + max(o["end_ms"] for o in r["ops"]) for r in recs)
        span = max(last - first, 1e-9)
        row = {"span_ms": span}
        for r in recs:
            row[f"rank{r['rank']}_busy"] = sum(o["end_ms"] - o["start_ms"] for o in r["ops"]) / span
        out[step] = row
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description="Merge per-rank step timelines into a trace and print rank utilisation")
    ap.add_argument("timeline_dir", help="<log_dir>/<run_id>/timeline")
    ap.add_argument("--out", default=None, help="write a chrome://tracing / Perfetto JSON here")
    a = ap.parse_args()
    records = load(a.timeline_dir)
    if a.out:
        with open(a.out, "w") as f:
            json.dump(chrome_trace(records), f)
    for step, row in utilisation(records).items():
        busy = " ".join(f"{k[:-5]}={v:.2f}" for k, v in row.items() if k.endswith("_busy"))
        print(f"step {step}: span {row['span_ms']:.1f} ms  busy: {busy}")


if __name__ == "__main__":
    main()
