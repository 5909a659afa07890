"""Checkpoints in the reference's directory layout, plus what resume needs.

Reference layout (src/ckpt.py:16-27,45-51), kept byte for byte for the model:

    <base_dir>/step_<N>/model.pt                 world_size == 1
    <base_dir>/step_<N>/model.<local_rank>.pt    world_size  > 1 (that rank's stage shard)

holding the stage's ``state_dict()`` (stage-local block indices).  The
reference never calls it from training and saves nothing else; real resume
needs more, so sibling files are added with the same suffix rule:

    optim[.<rank>].pt   inner optimiser state (+ scheduler step)
    outer[.<rank>].pt   DiLoCo global weights and Nesterov momentum of the stage
    meta.json           step, world shape, routing seed, config (written by the master)
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

import torch


class Checkpoint:
    def __init__(self, base_dir: str):
        self.base_dir = base_dir
        self.shard_id: Optional[int] = None
        os.makedirs(base_dir, exist_ok=True)

    def setup(self, world) -> None:
        if world.world_size > 1:
            self.shard_id = world.local_rank

    # -- paths -----------------------------------------------------------
    def _dir(self, step: int) -> str:
        return os.path.join(self.base_dir, f"step_{step}")

    def _name(self, stem: str = "model") -> str:
        return stem + (f".{self.shard_id}" if self.shard_id is not None else "") + ".pt"

    # -- reference API -----------------------------------------------------
    def save(self, step: int, model) -> str:
        d = self._dir(step)
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, self._name())
        sd = {k: v.detach().to("cpu") for k, v in model.state_dict().items()}
        torch.save(sd, path)
        return path

    def load(self, step: int) -> Dict[str, torch.Tensor]:
        d = self._dir(step)
        if not os.path.exists(d):
            raise ValueError(f"Checkpoint at step {step} does not exist")
        return self.load_from_dir(d)

    def load_from_dir(self, save_dir: str) -> Dict[str, torch.Tensor]:
        return torch.load(os.path.join(save_dir, self._name()), weights_only=True)

    def get_latest_step(self) -> Optional[int]:
        steps = []
        for d in os.listdir(self.base_dir):
            if d.startswith("step_"):
                try:
                    steps.append(int(d.split("_")[1]))
                except ValueError:
                    pass
        return max(steps) if steps else None

    # -- resume extras -------------------------------------------------------
    def save_extra(self, step: int, stem: str, obj: Dict[str, Any]) -> str:
        d = self._dir(step)
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, self._name(stem))
        torch.save(obj, path)
        return path

    def load_extra(self, step: int, stem: str) -> Optional[Dict[str, Any]]:
        path = os.path.join(self._dir(step), self._name(stem))
        if not os.path.exists(path):
            return None
        return torch.load(path, weights_only=False)

    def save_meta(self, step: int, meta: Dict[str, Any]) -> str:
        d = self._dir(step)
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, "meta.json")
        tmp = path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(meta, f, indent=1, default=str)
        os.replace(tmp, path)
        return path

    def load_meta(self, step: int) -> Optional[Dict[str, Any]]:
        path = os.path.join(self._dir(step), "meta.json")
        if not os.path.exists(path):
            return None
        with open(path) as f:
            return json.load(f)
