"""Reference arm of bench.py: the unmodified reference, timed on the same config.

The reference tree (``baseline/_ref/src``, installed offline from a copy of the
sources plus packaging metadata) is driven through its own entry point,
``src.train.main(SwarmConfig(...))``: its World (gloo + TCP store), its
threaded send/recv with host staging, its model, its optimisers, its DiLoCo
outer step on the host.  Nothing of this repository's engine, models or kernels
is on that path.  What the harness has to supply, because the box is offline
and two imports of the reference do not exist here:

* ``autorootcwd``                 an empty module (it only changes directory);
* ``pydantic_config.parse_argv``  not called (the config is built in Python),
                                   but the name must import;
* ``get_dataset`` / ``get_tokenizer`` in ``src.train``'s namespace return a
  seeded Zipf(1.0) token dataset of the named shape and a stand-in tokenizer
  instead of downloading from the Hugging Face hub.

Timing: ``src.train.train_step`` is wrapped (from outside, the function body is
untouched) with CUDA events after a device synchronize; the K steps after W
warm-up steps are summed, max over ranks.  The reference's own throughput
metric covers the same region (tokens / time spent in ``train_step``).
"""
from __future__ import annotations

import datetime
import json
import os
import socket
import sys
import tempfile
import time
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
TOPOLOGY = {1: 1, 2: 2, 4: 2, 8: 2}      # GPUs -> pipeline stages


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class _ZipfDataset:
    """Rows of seq_length + 1 token ids with an all-ones mask, in the interface
    the reference uses from a Hugging Face dataset."""

    def __init__(self, ids):
        self.ids = ids

    def __len__(self):
        return self.ids.shape[0]

    def __getitem__(self, i):
        row = self.ids[i]
        return {"input_ids": row.tolist(), "attention_mask": [1] * row.shape[0]}

    def select(self, idx):
        return _ZipfDataset(self.ids[list(idx)])

    def train_test_split(self, test_size, shuffle=True, seed=0):
        n = len(self)
        k = max(1, int(round(n * test_size)))
        return {"train": _ZipfDataset(self.ids[k:]), "test": _ZipfDataset(self.ids[:k])}


class _Tokenizer:
    eos_token_id = 50256
    eos_token = "<|endoftext|>"
    pad_token = "<|endoftext|>"

    def __len__(self):
        return 50257

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(i)) for i in ids)


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why}


def run_reference(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    if not os.path.isdir(os.path.join(REF, "src")):
        return _unavailable("baseline/_ref/src is missing: the offline install of the reference was not done") if rank == 0 else {}
    N = args.gpus
    if int(os.environ.get("WORLD_SIZE", "1")) != N:
        return _unavailable(f"--gpus {N} needs {N} ranks (launch with torch.distributed.run)") if rank == 0 else {}
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_WORLD_SIZE", "1"),
                 ("MASTER_ADDR", "127.0.0.1")):
        os.environ.setdefault(k, v)
    os.environ.setdefault("MASTER_PORT", str(_free_port()))
    os.environ["TOKENIZERS_PARALLELISM"] = "false"
    os.environ["WANDB_MODE"] = "disabled"

    sys.modules.setdefault("autorootcwd", types.ModuleType("autorootcwd"))
    try:
        import pydantic_config
        if not hasattr(pydantic_config, "parse_argv"):
            pydantic_config.parse_argv = lambda: {}
    except Exception as e:
        return _unavailable(f"pydantic_config not importable: {e}") if rank == 0 else {}
    sys.path.insert(0, REF)
    try:
        import torch
        import torch.distributed as dist
        import src.train as ref_train
    except Exception as e:
        return _unavailable(f"reference does not import here: {type(e).__name__}: {e}"[:300]) if rank == 0 else {}

    sys.path.insert(0, os.path.dirname(HERE))
    import bench as B
    from diloco_swarm_b200.utils.data import zipf_tokens   # data generator only (same tokens as our arm)

    S = TOPOLOGY.get(N, 2 if N % 2 == 0 else 1)
    K, W = args.steps, args.warmup
    H = max(1, min(50, K))
    total_steps = W + K
    n_rows = int(args.batch * (total_steps + 1) / 0.9) + 8

    ids = zipf_tokens(n_rows, args.seq + 1, 50257, 1.0, seed=0)
    ref_train.get_dataset = lambda cfg, split="train": _ZipfDataset(ids)
    ref_train.get_tokenizer = lambda: _Tokenizer()

    model_dims = {"tiny": (4, 4, 128), "small": (12, 12, 768), "medium": (24, 16, 1024), "large": (36, 20, 1280)}[args.model]
    if args.no_outer:
        # this image's pydantic_config turns the string "None" into None before validation, which the
        # reference's Literal["SGD", "AdamW", "None"] then refuses: build that one object without validation
        from src.config import OptimizerConfig
        outer = OptimizerConfig.model_construct(type="None", lr=0.0, nesterov=False, momentum=0.9, weight_decay=0.1,
                                                betas=[0.9, 0.95])
    else:
        outer = {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True}
    cfg = ref_train.SwarmConfig(
        model={"n_layer": model_dims[0], "n_head": model_dims[1], "n_embd": model_dims[2]},
        data={"path": "synthetic-zipf", "seq_length": args.seq, "num_workers": 0, "pin_memory": True},
        train={"max_steps": total_steps, "max_epochs": -1, "micro_batch_size": args.micro_batch,
               "batch_size": args.batch, "max_micro_batches": args.cap, "step_timeout": 3600.0,
               "inner_optimizer": {"type": "AdamW", "lr": 6e-4}, "outer_optimizer": outer,
               "scheduler": {"enable": True, "num_warmup_steps": 100}},
        swarm={"num_stages": S, "sync_every_n_steps": 1 if args.no_outer else H},
        eval={"enable": False}, sample={"enable": False},
        logging={"log_dir": os.path.join(tempfile.gettempdir(), "dswarm_ref_bench"), "run_id": f"ref{os.getpid()}",
                 "console": {"log_level": "ERROR"}, "file": {"log_level": "ERROR"}, "wandb": {"enable": False}},
    )

    step_ms = []
    losses = []
    stamps = []          # wall-clock (start, end) of every step, to pick the clock samples of the timed ones
    orig_step = ref_train.train_step

    def timed_step(step, *a, **kw):
        if not torch.cuda.is_available():          # CPU smoke runs of the harness only
            t0 = time.time()
            out = orig_step(step, *a, **kw)
            step_ms.append((time.time() - t0) * 1e3)
            losses.append(out[0].loss)
            return out
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = datetime.datetime.now()
        e0.record()
        out = orig_step(step, *a, **kw)
        e1.record()
        torch.cuda.synchronize()
        stamps.append((t0, datetime.datetime.now()))
        step_ms.append(e0.elapsed_time(e1))
        losses.append(out[0].loss)
        return out

    ref_train.train_step = timed_step
    sampler = None
    orig_loop = ref_train.train_loop

    def loop_with_clocks(*a, **kw):
        nonlocal sampler
        sampler = B.ClockSampler(rank == 0)
        return orig_loop(*a, **kw)

    ref_train.train_loop = loop_with_clocks
    # main() ends with destroy_process_group; the max over ranks has to happen before that
    result = {}
    orig_destroy = dist.destroy_process_group

    def reduce_then_destroy(*a, **kw):
        ms = torch.tensor([sum(step_ms[W:W + K])], dtype=torch.float64)
        if dist.get_world_size() > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        result["ms"] = float(ms.item())
        return orig_destroy(*a, **kw)

    dist.destroy_process_group = reduce_then_destroy
    try:
        ref_train.main(cfg)
    except Exception as e:
        return _unavailable(f"reference run failed: {type(e).__name__}: {e}"[:300]) if rank == 0 else {}
    finally:
        dist.destroy_process_group = orig_destroy
    windows = [(stamps[W][0], stamps[W + K - 1][1])] if len(stamps) >= W + K else []
    clocks = sampler.stop(windows) if (sampler is not None and rank == 0) else None
    if rank != 0 or "ms" not in result or len(step_ms) < W + K:
        return {}
    ms = result["ms"]
    tokens = args.batch * args.seq * K
    value = tokens / (ms / 1e3)
    R = N // S
    return {
        "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": N, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic Zipf(1.0) token ids, random-init weights", "impl": "reference",
        "config": {"model": f"gpt2-{args.model}", "global_batch": args.batch, "seq_len": args.seq,
                   "micro_batch": args.micro_batch, "parallelism": f"{S} stages x {R} replicas",
                   "algorithm": "swarm" if args.no_outer else f"diloco-swarm H={H}", "max_micro_batches": args.cap,
                   "transport": "gloo + host staging (the reference as shipped)",
                   "l2": "per-step working set (GBs) exceeds the 126 MB L2; no explicit flush"},
        "clocks": clocks,
        "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": ms / K,
                "note": "the reference's step always starts from host batches and reads the loss back"},
        "loss": losses[-1] if losses else None,
    }


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(HERE))
    import bench
    print(json.dumps(run_reference(bench.parse_args())))
