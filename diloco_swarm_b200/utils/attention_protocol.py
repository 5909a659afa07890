"""The hand-over protocol of ``attention_bwd_kernel`` (csrc/attention.cu) as a model for ``protocol_sim``.

Four roles and the barriers between them, in the order the kernel uses them.  One CTA walks ``items`` (a
list of step counts: an item is one kv tile of one (batch, head), a step one query tile against it).

  producer  K / V of item w into buffer w & 1 (waits kv_empty of the item two back), then one (Q, dO) pair
            per step into stage g % 2 (waits q_empty)
  mma       S / dP of step g+1 as soon as the rows have read the pair of step g (sdp_read), also for the first
            step of the next item (waits its kv_full); on pds_full: dV, dK, commit q_empty, wait dq_free of
            the step before, dQ, commit dq_full (and kv_empty on the item's last step)
  rows      wait sdp_full, read S / dP, arrive sdp_read, compute, wait dq_full of the step before (its
            products read P / dS) and, on an item's first step, dkv_stored of the item before (its dK / dV
            were staged in the P buffer), write P / dS, arrive pds_full, then take the dQ of the step before
            out of TMEM, wait for the staging tile, stage it, arrive dq_staged; after an item: read dK / dV,
            arrive dkv_free, stage them in the P buffer, arrive dkv_staged
  reducer   per step: wait dq_staged, bulk reduce-add out of the staging tile, arrive dq_stage_free; per
            item: wait dkv_staged, two bulk stores out of the P buffer, arrive dkv_stored

``drop`` names one wait or one ordering to leave out (a mutation): the tests use it to show that the checker
sees the race or the deadlock that the wait prevents.
"""
from __future__ import annotations

import random
from typing import Dict, List, Optional

from .protocol_sim import Barrier, Sim

MUTATIONS = ("rows_wait_dq_full", "mma_wait_sdp_read", "mma_wait_dq_free", "producer_wait_q_empty",
             "producer_wait_kv_empty", "rows_wait_dq_stage_free", "rows_wait_dkv_stored", "q_empty_before_dk")
# A wait of the kernel that the model shows to be implied by another: the issuer's wait for dkv_free before an
# item's first dV / dK products.  Those products also wait for pds_full of that step, at which the row threads
# arrive only after they have read the previous item's dK / dV (program order of the row threads).
IMPLIED = ("mma_wait_dkv_free",)


def run_attention_bwd(items: List[int], rng: random.Random, drop: Optional[str] = None) -> float:
    """Simulates one CTA; returns the finishing time in ns.  Raises ``Hazard`` or ``Deadlock``."""
    assert drop is None or drop in MUTATIONS + IMPLIED
    sim = Sim()
    B: Dict[str, Barrier] = {n: Barrier(n, 1) for n in (
        "kv_full0", "kv_full1", "kv_empty0", "kv_empty1", "q_full0", "q_full1", "q_empty0", "q_empty1",
        "sdp_full", "pds_full", "dq_full", "dq_free", "dkv_free", "sdp_read", "dq_staged", "dq_stage_free",
        "dkv_staged", "dkv_stored")}

    def lat(lo: float, hi: float) -> float:
        return rng.uniform(lo, hi)

    t_mma = lat(15, 70)             # one tcgen05.mma on the pipe
    t_issue = lat(30, 60)           # what issuing one costs the thread
    n_items = len(items)

    def producer():
        g = 0
        for w, steps in enumerate(items):
            kb = w & 1
            if drop != "producer_wait_kv_empty":
                yield ("wait", B[f"kv_empty{kb}"], ((w >> 1) & 1) ^ 1)
            yield ("copy", [], [(f"KV{kb}", w)], lat(300, 2500), B[f"kv_full{kb}"], None)
            for _ in range(steps):
                s = g % 2
                if drop != "producer_wait_q_empty":
                    yield ("wait", B[f"q_empty{s}"], ((g // 2) & 1) ^ 1)
                yield ("copy", [], [(f"QDO{s}", g)], lat(300, 2500), B[f"q_full{s}"], None)
                g += 1

    def issue_sdp(gs: int, wi: int, first: bool):
        if gs > 0 and drop != "mma_wait_sdp_read":
            yield ("wait", B["sdp_read"], (gs - 1) & 1)
        if first:
            yield ("wait", B[f"kv_full{wi & 1}"], (wi >> 1) & 1)
        yield ("wait", B[f"q_full{gs % 2}"], (gs // 2) & 1)
        yield ("mma", [(f"QDO{gs % 2}", gs), (f"KV{wi & 1}", wi)], [("S", gs)], 8 * t_mma)
        yield ("commit", B["sdp_full"])
        yield ("delay", 8 * t_issue)

    def mma():
        g = 0
        for w, steps in enumerate(items):
            kb = w & 1
            more = w + 1 < n_items
            if w == 0:
                yield from issue_sdp(0, 0, True)
            for it in range(steps):
                s = g % 2
                if it + 1 < steps:
                    yield from issue_sdp(g + 1, w, False)
                elif more:
                    yield from issue_sdp(g + 1, w + 1, True)
                yield ("wait", B["pds_full"], g & 1)
                if it == 0 and w > 0 and drop != "mma_wait_dkv_free":
                    yield ("wait", B["dkv_free"], (w - 1) & 1)
                yield ("mma", [("P", g), (f"QDO{s}", g)], ["DKV"], 8 * t_mma)            # dV
                if drop == "q_empty_before_dk":
                    yield ("commit", B[f"q_empty{s}"])
                yield ("mma", [("DS", g), (f"QDO{s}", g)], [("DKV", (w, it))], 8 * t_mma)   # dK
                if drop != "q_empty_before_dk":
                    yield ("commit", B[f"q_empty{s}"])
                yield ("delay", 16 * t_issue)
                if g > 0 and drop != "mma_wait_dq_free":
                    yield ("wait", B["dq_free"], (g - 1) & 1)
                yield ("mma", [("DS", g), (f"KV{kb}", w)], [("DQT", g)], 8 * t_mma)       # dQ
                yield ("commit", B["dq_full"])
                if it + 1 == steps:
                    yield ("commit", B[f"kv_empty{kb}"])
                yield ("delay", 8 * t_issue)
                g += 1

    def drain_dq(gs: int):
        yield ("delay", lat(0, 1500))                  # the row warps are not in step with the issuing thread
        yield ("wait", B["dq_full"], gs & 1)
        yield ("read", ("DQT", gs))
        yield ("delay", lat(50, 300))
        yield ("arrive", B["dq_free"])
        if gs > 0 and drop != "rows_wait_dq_stage_free":
            yield ("wait", B["dq_stage_free"], (gs - 1) & 1)
        yield ("write", ("STG", gs))
        yield ("delay", lat(50, 300))
        yield ("arrive", B["dq_staged"])

    def rows():
        g = 0
        for w, steps in enumerate(items):
            for it in range(steps):
                yield ("wait", B["sdp_full"], g & 1)
                yield ("read", ("S", g))
                yield ("delay", lat(100, 500))
                yield ("arrive", B["sdp_read"])
                yield ("delay", lat(300, 2000))
                if it > 0 and drop != "rows_wait_dq_full":
                    yield ("wait", B["dq_full"], (g - 1) & 1)
                if it == 0 and w > 0 and drop != "rows_wait_dkv_stored":
                    yield ("wait", B["dkv_stored"], (w - 1) & 1)
                yield ("write", ("DS", g))
                yield ("write", ("P", g))
                yield ("delay", lat(100, 700))
                yield ("arrive", B["pds_full"])
                if it > 0:
                    yield from drain_dq(g - 1)
                g += 1
            yield from drain_dq(g - 1)
            yield ("read", ("DKV", (w, steps - 1)))
            yield ("delay", lat(50, 300))
            yield ("arrive", B["dkv_free"])
            yield ("write", ("P", ("dkv", w)))         # dK / dV staged in the P buffer
            yield ("delay", lat(50, 300))
            yield ("arrive", B["dkv_staged"])

    def reducer():
        g = 0
        for w, steps in enumerate(items):
            for _ in range(steps):
                yield ("wait", B["dq_staged"], g & 1)
                done = Barrier(f"reduce{g}", 1)
                yield ("copy", [("STG", g)], [], lat(100, 1500), done, None)
                yield ("wait", done, 0)               # cp.async.bulk.wait_group.read
                yield ("arrive", B["dq_stage_free"])
                g += 1
            yield ("wait", B["dkv_staged"], w & 1)
            done = Barrier(f"store{w}", 1)
            yield ("copy", [("P", ("dkv", w))], [], lat(100, 1500), done, None)
            yield ("wait", done, 0)
            yield ("arrive", B["dkv_stored"])

    sim.add_role("producer", producer())
    sim.add_role("mma", mma())
    sim.add_role("rows", rows())
    sim.add_role("reducer", reducer())
    return sim.run()


FWD_MUTATIONS = ("rows_wait_o_full", "mma_wait_s_free", "producer_wait_kv_empty", "producer_wait_q_empty",
                 "rows_end_wait_o_full")
# Implied by p_full of the next item's first tile, at which the softmax rows arrive only after they have read
# the previous item's output rows.
FWD_IMPLIED = ("mma_wait_o_free",)


def run_attention_fwd(items: List[int], rng: random.Random, drop: Optional[str] = None) -> float:
    """``attention_fwd_kernel`` (csrc/attention.cu): one CTA walks ``items`` (kv tiles per query tile).

      producer  Q of item w (waits q_empty of the item before), then one (K, V) pair per kv tile into stage
                g & 1 (waits kv_empty)
      mma       S of tile g+1 as soon as the rows have read S of tile g (s_free), also the next item's first
                (waits its q_full); q_empty is committed with an item's last S; on p_full: P V into the output
                rows (waits o_free of the item before on an item's first tile), commit o_full and kv_empty
      rows      wait s_full, read S, arrive s_free, row maximum; from the item's second tile on wait o_full of
                the tile before (its product reads P and accumulates onto the rows that a rescale would touch),
                write P, arrive p_full; after an item: wait o_full of the last tile, read the output rows,
                arrive o_free
    """
    assert drop is None or drop in FWD_MUTATIONS + FWD_IMPLIED
    sim = Sim()
    B: Dict[str, Barrier] = {n: Barrier(n, 1) for n in (
        "q_full", "q_empty", "kv_full0", "kv_full1", "kv_empty0", "kv_empty1", "s_full", "s_free", "p_full", "o_full",
        "o_free")}

    def lat(lo: float, hi: float) -> float:
        return rng.uniform(lo, hi)

    t_mma = lat(15, 70)
    t_issue = lat(30, 60)
    n_items = len(items)

    def producer():
        g = 0
        for w, n_kv in enumerate(items):
            if w > 0 and drop != "producer_wait_q_empty":
                yield ("wait", B["q_empty"], (w - 1) & 1)
            yield ("copy", [], [("Q", w)], lat(300, 2500), B["q_full"], None)
            for _ in range(n_kv):
                s = g & 1
                if drop != "producer_wait_kv_empty":
                    yield ("wait", B[f"kv_empty{s}"], ((g >> 1) & 1) ^ 1)
                yield ("copy", [], [(f"KV{s}", g)], lat(300, 2500), B[f"kv_full{s}"], None)
                g += 1

    def issue_s(gt: int, wi: int, first: bool, last: bool):
        if first:
            yield ("wait", B["q_full"], wi & 1)
        yield ("wait", B[f"kv_full{gt & 1}"], (gt >> 1) & 1)
        yield ("mma", [("Q", wi), (f"KV{gt & 1}", gt)], [("S", gt)], 4 * t_mma)
        yield ("commit", B["s_full"])
        if last:
            yield ("commit", B["q_empty"])
        yield ("delay", 4 * t_issue)

    def mma():
        g = 0
        for w, n_kv in enumerate(items):
            nxt = items[w + 1] if w + 1 < n_items else 0
            if g == 0:
                yield from issue_s(0, 0, True, n_kv == 1)
            for j in range(n_kv):
                s = g & 1
                more = j + 1 < n_kv
                if more or nxt > 0:
                    if drop != "mma_wait_s_free":
                        yield ("wait", B["s_free"], g & 1)
                    if more:
                        yield from issue_s(g + 1, w, False, j + 2 == n_kv)
                    else:
                        yield from issue_s(g + 1, w + 1, True, nxt == 1)
                yield ("wait", B["p_full"], g & 1)
                if j == 0 and w > 0 and drop != "mma_wait_o_free":
                    yield ("wait", B["o_free"], (w - 1) & 1)
                yield ("mma", [("P", g), (f"KV{s}", g)], [("O", g)], 8 * t_mma)
                yield ("commit", B["o_full"])
                yield ("commit", B[f"kv_empty{s}"])
                yield ("delay", 8 * t_issue)
                g += 1

    def rows():
        g = 0
        for w, n_kv in enumerate(items):
            for j in range(n_kv):
                yield ("wait", B["s_full"], g & 1)
                yield ("read", ("S", g))
                yield ("delay", lat(100, 400))
                yield ("arrive", B["s_free"])
                yield ("delay", lat(100, 500))              # row maximum
                if j > 0:
                    if drop != "rows_wait_o_full":
                        yield ("wait", B["o_full"], (g - 1) & 1)
                    if rng.random() < 0.3:                    # the running maximum grew: rescale the output rows
                        yield ("read", ("O", g - 1))
                        yield ("write", ("O", g - 1))
                        yield ("delay", lat(100, 400))
                yield ("write", ("P", g))
                yield ("delay", lat(400, 1500))
                yield ("arrive", B["p_full"])
                g += 1
            if drop != "rows_end_wait_o_full":
                yield ("wait", B["o_full"], (g - 1) & 1)
            yield ("read", ("O", g - 1))
            yield ("delay", lat(50, 300))
            yield ("arrive", B["o_free"])
            yield ("delay", lat(100, 800))                    # normalise and store the rows

    sim.add_role("producer", producer())
    sim.add_role("mma", mma())
    sim.add_role("rows", rows())
    return sim.run()
