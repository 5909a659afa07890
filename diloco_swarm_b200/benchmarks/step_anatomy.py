"""Where one training step's device time goes, kernel by kernel, measured in place.

    python -m diloco_swarm_b200.benchmarks.step_anatomy [--model small --batch 64 --micro-batch 16 --steps 2]

Runs the 1-GPU engine through ``Trainer.train_step`` with every Python entry
point of ``ops/kernels.py`` and ``ops/attention.py`` bracketed by a pair of
CUDA events, everything on one stream (the weight-gradient side stream is
switched off so that intervals do not overlap), and prints the time per
(entry point, shape, epilogue) summed over the measured steps, with the
achieved TFLOP/s of the GEMMs.  Unlike a tight loop over one kernel, the
operands here are in whatever cache state the step leaves them in and the clocks
are those of the power-capped step.  The events add a little launch overhead;
this is a diagnosis tool, not a benchmark.
"""
from __future__ import annotations

import argparse
import collections
import json
import os

os.environ["DSWARM_WGRAD_STREAM"] = "0"

import torch  # noqa: E402

MODES = {0: "store", 1: "gelu", 2: "resid", 3: "mul", 4: "atomic_f32", 5: "store_f32"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="small")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--micro-batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args()

    from ..config import Config, load_toml
    from ..models import engine_b200 as E
    from ..ops import kernels as K
    from ..train import Trainer
    from ..utils import data as D

    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    cfg = Config(
        model=load_toml(os.path.join(root, "configs", "model", f"gpt2-{a.model}.toml")),
        data={"path": "synthetic:zipf", "seq_length": a.seq, "num_examples": a.batch * 2},
        train={"micro_batch_size": a.micro_batch, "batch_size": a.batch, "max_steps": 10 ** 6,
               "inner_optimizer": {"type": "AdamW", "lr": 6e-4}, "outer_optimizer": {"type": "None", "lr": 0.0}},
        swarm={"num_stages": 1}, eval={"enable": False}, sample={"enable": False},
        logging={"log_dir": "/tmp/dswarm_anatomy", "console": {"log_level": "ERROR"}, "file": {"log_level": "ERROR"}},
        engine="b200")
    tr = Trainer(cfg)
    tr.num_train_steps = 10 ** 6
    ds = D.get_dataset(cfg.data, D.ByteTokenizer(), seed=0)
    batch = {k: v.cuda() for k, v in D.collate(ds, 0, a.batch).items()}

    records = []
    recording = [False]

    def wrap(mod, name, label):
        fn = getattr(mod, name)

        def inner(*args, **kw):
            if not recording[0]:
                return fn(*args, **kw)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*args, **kw)
            e1.record()
            records.append((label(*args, **kw), e0, e1))
            return out
        setattr(mod, name, inner)

    def gemm_label(x, w, **kw):
        a_t, b_t = kw.get("a_t", False), kw.get("b_t", True)
        Kd, M = (x.shape if a_t else x.shape[::-1])
        N = w.shape[0] if b_t else w.shape[1]
        tag = MODES[kw.get("mode", 0)] + ("+bias" if kw.get("bias") is not None else "")
        return ("gemm", (M, N, Kd), ("tn" if a_t else ("nt" if b_t else "nn")) + " " + tag +
                (f" split{kw['split_k']}" if kw.get("split_k", 1) > 1 else ""))

    wrap(K, "gemm", gemm_label)
    for name in ("layernorm_fwd", "layernorm_bwd", "colsum_accum", "embedding_fwd", "embedding_bwd", "cross_entropy",
                 "grad_norm_and_clip", "adamw_step", "cast_to_bf16"):
        wrap(K, name, (lambda n: (lambda *args, **kw: (n, tuple(args[0].shape), "")))(name))
    wrap(E, "attention_fwd", lambda qkv, B, T, nh, **kw: ("attention_fwd", (B, T, nh), ""))
    wrap(E, "attention_bwd", lambda dout, ctx: ("attention_bwd", tuple(dout.shape), ""))

    for i in range(a.warmup):
        tr.train_step(i + 1, batch)
    torch.cuda.synchronize()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    recording[0] = True
    s0.record()
    for i in range(a.steps):
        tr.train_step(a.warmup + i + 1, batch)
    s1.record()
    torch.cuda.synchronize()
    recording[0] = False
    total = s0.elapsed_time(s1)
    agg = collections.OrderedDict()
    for label, e0, e1 in records:
        t = e0.elapsed_time(e1)
        cur = agg.setdefault(label, [0.0, 0])
        cur[0] += t
        cur[1] += 1
    covered = sum(v[0] for v in agg.values())
    rows = sorted(agg.items(), key=lambda kv: -kv[1][0])
    for (name, shape, tag), (ms, n) in rows:
        row = {"op": name, "shape": list(shape), "tag": tag, "calls": n, "ms_total": round(ms, 3),
               "us_per_call": round(1e3 * ms / n, 1), "share": round(ms / total, 4)}
        if name == "gemm":
            row["tflops"] = round(2.0 * shape[0] * shape[1] * shape[2] * n / ms / 1e9, 1)
        print(json.dumps(row))
    by_op = collections.defaultdict(float)
    for (name, _, _), (ms, _) in agg.items():
        by_op[name] += ms
    print(json.dumps({"steps": a.steps, "ms_per_step": round(total / a.steps, 2),
                      "covered_by_brackets": round(covered / total, 4),
                      "share_by_op": {k: round(v / total, 4) for k, v in sorted(by_op.items(), key=lambda kv: -kv[1])}}))


if __name__ == "__main__":
    main()
