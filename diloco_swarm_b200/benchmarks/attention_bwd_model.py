"""Step time of ``attention_bwd_kernel`` from its hand-over protocol and a handful of measured latencies.

    python -m diloco_swarm_b200.benchmarks.attention_bwd_model

The kernel (csrc/attention.cu) is four roles that hand buffers to one another through mbarriers; its step
time is the length of the longest chain of waits through them, which no counter shows.  This tool replays the
protocol in ``utils/protocol_sim`` with the latencies read off the in-kernel timeline
(``benchmarks/timelines.py``: a tcgen05.mma costs the issuing thread 52 ns, a (Q, dO) reload takes 1.1 us from
the release of its stage to the data, the row threads need 0.3 us to take S / dP out of TMEM, 0.85 us for the
row algebra, 0.4 us to write P / dS, 0.45 us to hand dQ over) and prints the step time for the kernel as it
is and for a list of what-ifs, so that a change can be judged before it is written.  No GPU is involved; the
reference has no counterpart.
"""
from __future__ import annotations

import argparse
from typing import Dict, List

from ..utils.protocol_sim import Barrier, Sim

MEASURED = dict(t_mma=45.0, t_issue=52.0, tma=1100.0, ld=300.0, compute=850.0, write=400.0, drain_ld=200.0,
                drain_st=250.0, reduce=600.0, qstages=2, early=True)


def step_time(items: List[int], P: Dict[str, float]) -> float:
    """ns per step for one CTA that walks ``items`` (steps per work item) with the latencies ``P``."""
    sim = Sim()
    QS = int(P["qstages"])
    names = ["kv_full0", "kv_full1", "kv_empty0", "kv_empty1", "sdp_full", "pds_full", "dq_full", "dq_free",
             "sdp_read", "dq_staged", "dq_stage_free", "dkv_staged", "dkv_stored"]
    names += [f"q_full{i}" for i in range(QS)] + [f"q_empty{i}" for i in range(QS)]
    B = {n: Barrier(n, 1) for n in names}
    t_mma, t_issue = P["t_mma"], P["t_issue"]
    n_items = len(items)

    def producer():
        g = 0
        for w, steps in enumerate(items):
            kb = w & 1
            yield ("wait", B[f"kv_empty{kb}"], ((w >> 1) & 1) ^ 1)
            yield ("copy", [], [], P["tma"], B[f"kv_full{kb}"], None)
            for _ in range(steps):
                s = g % QS
                yield ("wait", B[f"q_empty{s}"], ((g // QS) & 1) ^ 1)
                yield ("copy", [], [], P["tma"], B[f"q_full{s}"], None)
                g += 1

    def issue_sdp(gs, wi, first):
        if gs > 0:
            yield ("wait", B["sdp_read"], (gs - 1) & 1)
        if first:
            yield ("wait", B[f"kv_full{wi & 1}"], (wi >> 1) & 1)
        yield ("wait", B[f"q_full{gs % QS}"], (gs // QS) & 1)
        yield ("mma", [], [], 8 * t_mma)
        yield ("commit", B["sdp_full"])
        yield ("delay", 8 * t_issue)

    def next_pair(g, w, it, steps):
        if it + 1 < steps:
            yield from issue_sdp(g + 1, w, False)
        elif w + 1 < n_items:
            yield from issue_sdp(g + 1, w + 1, True)

    def mma():
        g = 0
        for w, steps in enumerate(items):
            if w == 0:
                yield from issue_sdp(0, 0, True)
            for it in range(steps):
                s = g % QS
                if P["early"]:
                    yield from next_pair(g, w, it, steps)
                yield ("wait", B["pds_full"], g & 1)
                if not P["early"]:
                    yield from next_pair(g, w, it, steps)
                yield ("mma", [], [], 16 * t_mma)                 # dV, dK
                yield ("commit", B[f"q_empty{s}"])
                yield ("delay", 16 * t_issue)
                if g > 0:
                    yield ("wait", B["dq_free"], (g - 1) & 1)
                yield ("mma", [], [], 8 * t_mma)                  # dQ
                yield ("commit", B["dq_full"])
                if it + 1 == steps:
                    yield ("commit", B[f"kv_empty{w & 1}"])
                yield ("delay", 8 * t_issue)
                g += 1

    def drain(gs):
        yield ("wait", B["dq_full"], gs & 1)
        yield ("delay", P["drain_ld"])
        yield ("arrive", B["dq_free"])
        if gs > 0:
            yield ("wait", B["dq_stage_free"], (gs - 1) & 1)
        yield ("delay", P["drain_st"])
        yield ("arrive", B["dq_staged"])

    def rows():
        g = 0
        for w, steps in enumerate(items):
            for it in range(steps):
                yield ("wait", B["sdp_full"], g & 1)
                yield ("delay", P["ld"])
                yield ("arrive", B["sdp_read"])
                yield ("delay", P["compute"])
                if it > 0:
                    yield ("wait", B["dq_full"], (g - 1) & 1)
                if it == 0 and w > 0:
                    yield ("wait", B["dkv_stored"], (w - 1) & 1)
                yield ("delay", P["write"])
                yield ("arrive", B["pds_full"])
                if it > 0:
                    yield from drain(g - 1)
                g += 1
            yield from drain(g - 1)
            yield ("delay", 250.0)                                # dK / dV out of TMEM into the P buffer
            yield ("arrive", B["dkv_staged"])

    def reducer():
        g = 0
        for w, steps in enumerate(items):
            for _ in range(steps):
                yield ("wait", B["dq_staged"], g & 1)
                yield ("delay", P["reduce"])
                yield ("arrive", B["dq_stage_free"])
                g += 1
            yield ("wait", B["dkv_staged"], w & 1)
            yield ("delay", P["reduce"])
            yield ("arrive", B["dkv_stored"])

    for name, role in (("producer", producer), ("mma", mma), ("rows", rows), ("reducer", reducer)):
        sim.add_role(name, role())
    return sim.run() / sum(items)


WHAT_IFS = [
    ("the kernel as it is", {}),
    ("next S / dP pair only after the hand-over (the earlier build)", {"early": False}),
    ("three (Q, dO) stages instead of two", {"qstages": 3}),
    ("(Q, dO) reload in 0.6 us (L2 hit)", {"tma": 600.0}),
    ("MMA issue at half the cost (two issuing threads, or M = 256 products of a CTA pair)", {"t_issue": 26.0, "t_mma": 30.0}),
    ("row algebra in 0.6 us", {"compute": 600.0}),
    ("P / dS written in 0.2 us", {"write": 200.0}),
    ("dQ hand-over in 0.2 us", {"drain_ld": 100.0, "drain_st": 100.0}),
    ("S / dP out of TMEM in 0.1 us", {"ld": 100.0}),
]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--items", default="8,5,5,2,2,7,7,4,4,1,1",
                    help="steps per work item of one CTA (T = 1024: a kv tile meets 1 to 8 query tiles)")
    a = ap.parse_args()
    items = [int(x) for x in a.items.split(",")]
    for name, over in WHAT_IFS:
        P = dict(MEASURED)
        P.update(over)
        print(f"{step_time(items, P):7.0f} ns per step   {name}")


if __name__ == "__main__":
    main()
