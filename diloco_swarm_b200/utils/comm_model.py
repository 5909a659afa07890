"""Analytic communication volume of a SWARM / DiLoCo-SWARM run.

The reference's results notebook estimates bytes moved per step with two
closed forms (notebooks/3.0-results.ipynb, cell 16): pipeline traffic
``2 (S-1) B T d bytes_per_value`` (activations forward, gradients backward over
every stage boundary) and data-parallel traffic of a ring all-reduce of each
stage's parameters, paid on sync steps only.  This module restates them and
adds the figures for this framework's wire formats (bf16 pipeline payload with
no metadata plane; fused all-reduce over peer memory where every replica reads
and writes (R-1)/R of the buffer).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List


def pp_bytes_per_step(num_stages: int, batch_size: int, seq_length: int, hidden_dim: int,
                      bytes_per_value: int = 4, metadata_plane: bool = False) -> float:
    """Bytes crossing stage boundaries per step for the whole batch.  With
    ``metadata_plane`` every message is doubled, as the reference's serializer
    does (src/serializer.py:9-15)."""
    b = 2.0 * (num_stages - 1) * batch_size * seq_length * hidden_dim * bytes_per_value
    return 2.0 * b if metadata_plane else b


def dp_bytes_per_sync(num_stages: int, replicas_per_stage: int, num_params: float, bytes_per_param: int = 4) -> float:
    """Bytes one replica of every stage sends for a ring all-reduce of its stage's
    parameters: 2 (R-1)/R of the stage, summed over the S stages (the notebook's
    convention: 1.08 GB for GPT-2 small, 2 stages x 4 replicas)."""
    R = replicas_per_stage
    if R <= 1:
        return 0.0
    per_stage = num_params / num_stages * bytes_per_param
    return num_stages * 2.0 * (R - 1) / R * per_stage


@dataclass
class CommCost:
    pp_per_step: float
    dp_per_sync: float
    syncs: int
    steps: int

    @property
    def total(self) -> float:
        return self.pp_per_step * self.steps + self.dp_per_sync * self.syncs


def run_cost(steps: int, num_stages: int, replicas_per_stage: int, batch_size: int, seq_length: int, hidden_dim: int,
             num_params: float, sync_every_n_steps: int = 1, pp_bytes_per_value: int = 4, dp_bytes_per_param: int = 4,
             metadata_plane: bool = False) -> CommCost:
    syncs = steps // max(1, sync_every_n_steps) + (1 if steps % max(1, sync_every_n_steps) else 0)
    return CommCost(pp_bytes_per_step(num_stages, batch_size, seq_length, hidden_dim, pp_bytes_per_value, metadata_plane),
                    dp_bytes_per_sync(num_stages, replicas_per_stage, num_params, dp_bytes_per_param), syncs, steps)


def cumulative(cost: CommCost, sync_every_n_steps: int) -> List[float]:
    """Cumulative bytes after each step (the curve the notebook plots against perplexity)."""
    out, acc = [], 0.0
    for step in range(1, cost.steps + 1):
        acc += cost.pp_per_step
        if step % max(1, sync_every_n_steps) == 0 or step == cost.steps:
            acc += cost.dp_per_sync
        out.append(acc)
    return out


def summary(model: str = "small") -> Dict[str, float]:
    """The notebook's headline comparison for GPT-2 small, 2 stages x 4 replicas, batch 2048."""
    dims = {"small": (180e6, 768), "medium": (405e6, 1024), "large": (800e6, 1280), "xl": (1500e6, 1600)}[model]
    swarm = run_cost(2000, 2, 4, 2048, 1024, dims[1], dims[0], 1)
    diloco = run_cost(2000, 2, 4, 2048, 1024, dims[1], dims[0], 50)
    return {"pp_gb_per_step": swarm.pp_per_step / 1e9, "dp_gb_per_sync": swarm.dp_per_sync / 1e9,
            "swarm_total_tb": swarm.total / 1e12, "diloco_swarm_total_tb": diloco.total / 1e12}
