"""Runs the reference's own ``src.train.main`` on CPU for a few steps (helper of test_reference_parity.py,
started under torch.distributed.run; not a test itself).

Same shims as the benchmark's reference arm (baseline/run_reference.py): an empty ``autorootcwd``, an unused
``parse_argv`` name, and a token matrix from a file in place of the hub dataset.  Everything else is the
reference's stock path.  Before the first step every rank saves the weights it starts from, so that this
framework can start from the same ones.
"""
import argparse
import os
import sys
import types

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--stages", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--mbs", type=int, default=2)
    ap.add_argument("--seq", type=int, default=32)
    ap.add_argument("--H", type=int, default=1)
    ap.add_argument("--outer", default="None", choices=["None", "nesterov"])
    ap.add_argument("--eval-size", type=float, default=0.1)
    ap.add_argument("--eval-every", type=int, default=0, help="0 = no evaluation")
    a = ap.parse_args()

    from baseline.run_reference import REF, _Tokenizer, _ZipfDataset
    sys.modules.setdefault("autorootcwd", types.ModuleType("autorootcwd"))
    import pydantic_config
    if not hasattr(pydantic_config, "parse_argv"):
        pydantic_config.parse_argv = lambda: {}
    sys.path.insert(0, REF)
    import src.train as ref_train

    ids = torch.from_numpy(np.load(a.tokens).astype(np.int64))
    ref_train.get_dataset = lambda cfg, split="train": _ZipfDataset(ids)
    ref_train.get_tokenizer = lambda: _Tokenizer()
    rank = int(os.environ.get("RANK", "0"))
    os.makedirs(a.out, exist_ok=True)
    stock_loop = ref_train.train_loop

    def save_start_then_train(num_train_steps, inner_model, *rest, **kw):
        torch.save({k: v.detach().clone() for k, v in inner_model.state_dict().items()},
                   os.path.join(a.out, f"w0.{rank}.pt"))
        return stock_loop(num_train_steps, inner_model, *rest, **kw)

    ref_train.train_loop = save_start_then_train
    # the reference draws the next-stage replica with Python's unseeded `random`; a seed per process makes
    # the probe's runs repeatable (which replica serves a microbatch does not change the gradients)
    import random
    random.seed(1000 + rank)
    if a.outer == "None":
        # this image's pydantic_config turns the string "None" into None before validation, which the
        # reference's Literal["SGD", "AdamW", "None"] then refuses: build that one object without validation
        from src.config import OptimizerConfig
        outer = OptimizerConfig.model_construct(type="None", lr=0.0, nesterov=False, momentum=0.9, weight_decay=0.1,
                                                betas=[0.9, 0.95])
    else:
        outer = {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True}
    cfg = ref_train.SwarmConfig(
        model={"n_layer": 4, "n_head": 4, "n_embd": 128},
        data={"path": "tokens-from-file", "seq_length": a.seq, "num_workers": 0, "pin_memory": False},
        train={"max_steps": a.steps, "max_epochs": -1, "micro_batch_size": a.mbs, "batch_size": a.batch,
               "max_micro_batches": 2, "inner_optimizer": {"type": "AdamW", "lr": 6e-4}, "outer_optimizer": outer},
        device="cpu", amp={"enable": False}, swarm={"num_stages": a.stages, "sync_every_n_steps": a.H},
        eval={"enable": a.eval_every > 0, "every_n_steps": a.eval_every if a.eval_every > 0 else -1, "eval_size": a.eval_size}, sample={"enable": False},
        logging={"log_dir": a.out, "run_id": "ref", "console": {"log_level": "ERROR"}, "wandb": {"enable": False}})
    ref_train.main(cfg)


if __name__ == "__main__":
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    os.environ["WANDB_MODE"] = "disabled"
    main()
