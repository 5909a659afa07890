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

A checkpoint can move to another topology: ``merge_model`` joins the stage shards into one state dict
with global block numbers (the file a one-process run loads), ``split_model`` cuts a whole model into
stage shards, ``reshard`` does both between two checkpoint directories:

    python -m diloco_swarm_b200.utils.ckpt --src logs/run/checkpoints/step_100 --dst out/step_100 \
        --num-stages 1                      # 8 GPUs of training -> one file for sampling on one GPU

Only the weights move; optimiser and DiLoCo state are tied to the old layout and start afresh.
"""
from __future__ import annotations

import json
import os
import re
from typing import Any, Dict, List, Optional, Sequence

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


# ---------------------------------------------------------------------- moving between topologies
_BLOCK_KEY = re.compile(r"^transformer\.h\.(\d+)\.(.+)$")


def _shard_path(step_dir: str, rank: int, world_size: int, stem: str = "model") -> str:
    return os.path.join(step_dir, f"{stem}.pt" if world_size == 1 else f"{stem}.{rank}.pt")


def _stage_layers(model_cfg: Dict[str, Any], num_stages: int, layer_split: str) -> List[List[int]]:
    from ..models.gpt2 import split_layers
    return split_layers(int(model_cfg["n_layer"]), num_stages, layer_split, int(model_cfg["n_embd"]),
                        int(model_cfg.get("vocab_size", 50304)))


def merge_model(step_dir: str, average_replicas: bool = False) -> Dict[str, torch.Tensor]:
    """The whole model of a checkpoint as one state dict with global block indices.  Each stage is
    read from its leader (rank = stage index); ``average_replicas`` takes the mean over the stage's
    replicas instead, which matters only for a checkpoint taken between two synchronisations."""
    with open(os.path.join(step_dir, "meta.json")) as f:
        meta = json.load(f)
    W, S = int(meta["world_size"]), int(meta["num_stages"])
    cfg = meta["config"]
    layers = _stage_layers(cfg["model"], S, cfg["swarm"].get("layer_split", "even"))
    full: Dict[str, torch.Tensor] = {}
    for s in range(S):
        ranks = [r for r in range(W) if r % S == s]
        shards = [torch.load(_shard_path(step_dir, r, W), weights_only=True)
                  for r in (ranks if average_replicas else ranks[:1])]
        for key, value in shards[0].items():
            if len(shards) > 1:
                value = torch.stack([sd[key].float() for sd in shards]).mean(0).to(value.dtype)
            m = _BLOCK_KEY.match(key)
            full[f"transformer.h.{layers[s][int(m.group(1))]}.{m.group(2)}" if m else key] = value
    return full


def split_model(full: Dict[str, torch.Tensor], stage_layers: Sequence[Sequence[int]], tied: bool = False
                ) -> List[Dict[str, torch.Tensor]]:
    """Stage shards (stage-local block indices, embeddings on the first stage, final LayerNorm and head
    on the last) of a whole-model state dict.  ``tied``: the model shares the embedding with the head
    (``parameter_sharing``), which only a one-stage model can do: it then has no separate head tensor."""
    S = len(stage_layers)
    where = {g: (s, li) for s, layers in enumerate(stage_layers) for li, g in enumerate(layers)}
    out: List[Dict[str, torch.Tensor]] = [{} for _ in range(S)]
    for key, value in full.items():
        m = _BLOCK_KEY.match(key)
        if m:
            s, li = where[int(m.group(1))]
            out[s][f"transformer.h.{li}.{m.group(2)}"] = value
        elif key.startswith("transformer.wte.") or key.startswith("transformer.wpe."):
            out[0][key] = value
        else:                                   # transformer.ln_f.*, lm_head.weight
            out[S - 1][key] = value
    if "lm_head.weight" not in out[S - 1] and "transformer.wte.weight" in full:
        # tied in a one-stage checkpoint: the last stage of a deeper pipeline holds its own copy
        if S > 1:
            out[S - 1]["lm_head.weight"] = full["transformer.wte.weight"].clone()
    if tied and S == 1:
        out[0].pop("lm_head.weight", None)      # the copy a deeper pipeline kept on its last stage
    return out


def reshard(src_step_dir: str, dst_step_dir: str, num_stages: int, replicas: int = 1, layer_split: str = "even",
            average_replicas: bool = False) -> Dict[str, Any]:
    """Rewrite the model of ``src_step_dir`` for ``num_stages`` x ``replicas`` ranks into ``dst_step_dir``
    (same file naming, ``meta.json`` updated).  Returns the new meta."""
    with open(os.path.join(src_step_dir, "meta.json")) as f:
        meta = json.load(f)
    full = merge_model(src_step_dir, average_replicas)
    layers = _stage_layers(meta["config"]["model"], num_stages, layer_split)
    shards = split_model(full, layers, tied=bool(meta["config"]["model"].get("parameter_sharing", False)))
    W = num_stages * replicas
    os.makedirs(dst_step_dir, exist_ok=True)
    for r in range(W):
        torch.save(shards[r % num_stages], _shard_path(dst_step_dir, r, W))
    new = dict(meta)
    new.update({"world_size": W, "num_stages": num_stages, "resharded_from": {
        "world_size": meta["world_size"], "num_stages": meta["num_stages"], "dir": os.path.abspath(src_step_dir)}})
    new["config"] = json.loads(json.dumps(meta["config"]))
    new["config"]["swarm"]["num_stages"] = num_stages
    new["config"]["swarm"]["layer_split"] = layer_split
    tmp = os.path.join(dst_step_dir, "meta.json.tmp")
    with open(tmp, "w") as f:
        json.dump(new, f, indent=1, default=str)
    os.replace(tmp, os.path.join(dst_step_dir, "meta.json"))
    return new


def _main() -> None:
    import argparse
    ap = argparse.ArgumentParser(description="Move a checkpoint's weights to another number of stages / replicas")
    ap.add_argument("--src", required=True, help="checkpoint directory .../checkpoints/step_<N>")
    ap.add_argument("--dst", required=True, help="output directory (a step_<N> directory of the new run)")
    ap.add_argument("--num-stages", type=int, required=True)
    ap.add_argument("--replicas", type=int, default=1)
    ap.add_argument("--layer-split", default="even")
    ap.add_argument("--average-replicas", action="store_true")
    a = ap.parse_args()
    meta = reshard(a.src, a.dst, a.num_stages, a.replicas, a.layer_split, a.average_replicas)
    print(f"wrote {meta['world_size']} shard(s) for {a.num_stages} stage(s) x {a.replicas} replica(s) to {a.dst}")


if __name__ == "__main__":
    _main()
