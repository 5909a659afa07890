"""Sample text from a checkpoint in one process.

    python -m diloco_swarm_b200.generate --ckpt logs/<run>/checkpoints/step_<N> --prompt "I am" \
        --max-new-tokens 40 --temperature 0.8 --top-k 20 --num-samples 3 [--device cuda]

The checkpoint may come from any topology: its stage shards are merged into the whole model
(utils/ckpt.py), which then runs the reference's single-process sampler (GPT2.generate,
src/model.py:160-175) on library ops.  The training command samples through the pipeline instead
(``Trainer.sample_loop``); this entry point is for using a trained model afterwards.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import List, Optional

import torch

from .models.gpt2 import GPT2Config, TorchStage
from .utils import ckpt as C
from .utils import data as D


def load_model(step_dir: str, device: str = "cpu", average_replicas: bool = False) -> TorchStage:
    """The whole model of the checkpoint in ``step_dir`` (a ``step_<N>`` directory with ``meta.json``)."""
    with open(os.path.join(step_dir, "meta.json")) as f:
        mc = json.load(f)["config"]["model"]
    cfg = GPT2Config(block_size=mc["block_size"], vocab_size=mc["vocab_size"], n_layer=mc["n_layer"],
                     n_head=mc["n_head"], n_embd=mc["n_embd"], dropout=mc.get("dropout", 0.0),
                     bias=mc.get("bias", True), parameter_sharing=mc.get("parameter_sharing", False))
    model = TorchStage(cfg, 0, 1)
    full = C.merge_model(step_dir, average_replicas)
    if cfg.parameter_sharing:
        full.pop("lm_head.weight", None)        # tied: the head is the embedding
        full["lm_head.weight"] = full["transformer.wte.weight"]
    model.load_state_dict(full)
    return model.to(device).eval()


@torch.no_grad()
def generate(model: TorchStage, tokenizer, prompt: str, max_new_tokens: int = 20, temperature: float = 1.0,
             top_k: Optional[int] = 20, num_samples: int = 1, seed: int = 0) -> List[str]:
    device = next(model.parameters()).device
    ids = D.tokenize(prompt, tokenizer)["input_ids"].repeat(num_samples, 1).to(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    out = model.generate(ids, max_new_tokens, temperature=temperature, top_k=top_k,
                         eos_token_id=tokenizer.eos_token_id, generator=gen)
    return [tokenizer.decode(row, skip_special_tokens=True) for row in out.cpu()]


def main() -> None:
    ap = argparse.ArgumentParser(description="Sample text from a checkpoint of any topology, in one process")
    ap.add_argument("--ckpt", required=True, help="checkpoint directory .../checkpoints/step_<N>")
    ap.add_argument("--prompt", default="I am")
    ap.add_argument("--max-new-tokens", type=int, default=20)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=20)
    ap.add_argument("--num-samples", type=int, default=5)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--average-replicas", action="store_true")
    a = ap.parse_args()
    model = load_model(a.ckpt, a.device, a.average_replicas)
    tokenizer = D.get_tokenizer()
    for i, text in enumerate(generate(model, tokenizer, a.prompt, a.max_new_tokens, a.temperature, a.top_k,
                                      a.num_samples, a.seed), start=1):
        print(f"Sample {i}: {text}")


if __name__ == "__main__":
    main()
