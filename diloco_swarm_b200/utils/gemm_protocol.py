"""The hand-over protocol of the persistent GEMM kernels (csrc/gemm_kernels.cuh) as a model for ``protocol_sim``.

Three roles per CTA (or CTA pair; the pair's barriers are modelled as one CTA's, the two halves arriving
together):

  producer  per tile and k-block group: wait empty[s] (phase of the ring's previous lap), load A and B into
            stage s = it % NSTAGE, completion on full[s]
  mma       per tile: wait acc_empty[tile & 1] (the epilogue has drained that accumulator two tiles ago); per
            k-block group: wait full[s], products into the accumulator, commit empty[s]; after the tile's last
            group commit acc_full[tile & 1]
  epilogue  per tile: wait acc_full[tile & 1], read the accumulator, arrive acc_empty[tile & 1], write the
            tile out

``drop`` leaves one wait out (a mutation), as in ``attention_protocol``.
"""
from __future__ import annotations

import random
from typing import Dict, List, Optional

from .protocol_sim import Barrier, Sim

MUTATIONS = ("producer_wait_empty", "mma_wait_full", "mma_wait_acc_empty", "epilogue_wait_acc_full")


def run_gemm(tiles: int, kgroups: int, nstage: int, rng: random.Random, drop: Optional[str] = None) -> float:
    assert drop is None or drop in MUTATIONS
    sim = Sim()
    B: Dict[str, Barrier] = {}
    for s in range(nstage):
        B[f"full{s}"] = Barrier(f"full{s}", 1)
        B[f"empty{s}"] = Barrier(f"empty{s}", 1)
    for b in range(2):
        B[f"acc_full{b}"] = Barrier(f"acc_full{b}", 1)
        B[f"acc_empty{b}"] = Barrier(f"acc_empty{b}", 1)

    def lat(lo: float, hi: float) -> float:
        return rng.uniform(lo, hi)

    t_group = lat(100, 500)             # the products of one k-block group on the pipe

    def producer():
        it = 0
        for t in range(tiles):
            for k in range(kgroups):
                s, ph = it % nstage, (it // nstage) & 1
                if drop != "producer_wait_empty":
                    yield ("wait", B[f"empty{s}"], ph ^ 1)
                yield ("copy", [], [(f"ST{s}", (t, k))], lat(300, 2000), B[f"full{s}"], None)
                it += 1

    def mma():
        it = 0
        for t in range(tiles):
            ab, aph = t & 1, (t >> 1) & 1
            if drop != "mma_wait_acc_empty":
                yield ("wait", B[f"acc_empty{ab}"], aph ^ 1)
            for k in range(kgroups):
                s, ph = it % nstage, (it // nstage) & 1
                if drop != "mma_wait_full":
                    yield ("wait", B[f"full{s}"], ph)
                yield ("mma", [(f"ST{s}", (t, k))], [(f"ACC{ab}", (t, k))], t_group)
                yield ("commit", B[f"empty{s}"])
                yield ("delay", lat(50, 400))
                it += 1
            yield ("commit", B[f"acc_full{ab}"])

    def epilogue():
        for t in range(tiles):
            ab, aph = t & 1, (t >> 1) & 1
            if drop != "epilogue_wait_acc_full":
                yield ("wait", B[f"acc_full{ab}"], aph)
            yield ("read", (f"ACC{ab}", (t, kgroups - 1)))
            yield ("delay", lat(300, 3000))
            yield ("arrive", B[f"acc_empty{ab}"])
            yield ("delay", lat(100, 1500))

    sim.add_role("producer", producer())
    sim.add_role("mma", mma())
    sim.add_role("epilogue", epilogue())
    return sim.run()
