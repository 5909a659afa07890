"""Communication-frequency sweep of DiLoCo-SWARM: the sync interval H against throughput, outer-sync cost and loss.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        -m diloco_swarm_b200.benchmarks.h_sweep --stages 2 --H 1,10,50,100,500 --steps 100

The reference sweeps H over {10, 20, 50, 100, 200} for 2 000 steps and reports validation perplexity
(experiments/experiment2.sh:3); its H = 1 run did not converge (experiments/experiment2.sh:135).  This tool runs,
in one process group and from the same seeded initial weights and the same seeded Zipf(1.0) batches, ``--steps``
training steps per value of H (GPT-2 small, global batch 512 x 1024, microbatch 16, inner AdamW 6e-4 with 100
warm-up steps, outer SGD-Nesterov lr 0.7 momentum 0.9; the last step always synchronises, as in the reference,
src/train.py:248) and prints one JSON line per H:

  tokens_per_s           B * T * steps / device time of the steps (CUDA events, max over ranks)
  outer_sync_ms          device time of the fused outer sync + bf16 refresh, mean over the steps that ran one,
                         max over ranks; outer_wait_ms is the wait for the slowest replica in front of it
  exposed_share          (outer_sync_ms + outer_wait_ms) * syncs / total time
  loss                   the training loss every ``--loss-every`` steps (mean over the last stage's replicas)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--stages", type=int, default=2)
    ap.add_argument("--H", default="1,10,50,100,500")
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3, help="untimed steps before each H (on a throw-away trainer state)")
    ap.add_argument("--model", default="small")
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--micro-batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--cap", type=int, default=8)
    ap.add_argument("--loss-every", type=int, default=10)
    ap.add_argument("--collective", default="fused")
    a = ap.parse_args()

    from ..config import Config, load_toml
    from ..train import Trainer
    from ..utils import data as D

    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

    def config(H: int) -> Config:
        return Config(
            model=load_toml(os.path.join(root, "configs", "model", f"gpt2-{a.model}.toml")),
            data={"path": "synthetic:zipf", "seq_length": a.seq, "num_examples": a.batch * 4, "pin_memory": True},
            train={"micro_batch_size": a.micro_batch, "batch_size": a.batch, "max_steps": 10 ** 6,
                   "max_micro_batches": a.cap, "step_timeout": 600,
                   "inner_optimizer": {"type": "AdamW", "lr": 6e-4},
                   "outer_optimizer": {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True},
                   "scheduler": {"enable": True, "num_warmup_steps": 100, "type": "cosine"}},
            swarm={"num_stages": a.stages, "sync_every_n_steps": H, "layer_split": "balanced", "collective": a.collective},
            eval={"enable": False}, sample={"enable": False},
            logging={"log_dir": "/tmp/dswarm_h_sweep", "run_id": f"H{H}_{os.getpid()}",
                     "console": {"log_level": "ERROR"}, "file": {"log_level": "ERROR"}},
            engine="b200")

    world = None
    for H in [int(x) for x in a.H.split(",")]:
        cfg = config(H)
        tr = Trainer(cfg, world=world)
        world = tr.world
        tr.num_train_steps = a.warmup + a.steps
        dev = tr.device
        ds = D.get_dataset(cfg.data, D.ByteTokenizer(), seed=0)
        batches = [{k: v.to(dev) for k, v in D.collate(ds, i * a.batch, (i + 1) * a.batch).items()} for i in range(4)]
        n_last = len(world.last_stage_ranks)
        syncs, losses = [], []
        for s in range(1, a.warmup + 1):
            tr.train_step(s, batches[s % 4])
        world.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(a.warmup + 1, a.warmup + a.steps + 1):
            before = tr.last_sync_phase_ms
            local, _ = tr.train_step(s, batches[s % 4])
            if tr.last_sync_phase_ms is not before:
                syncs.append(tr.last_sync_phase_ms)
            if (s - a.warmup) % a.loss_every == 0 or s == a.warmup + a.steps:
                losses.append((s - a.warmup, local.loss if tr.engine.is_last else 0.0))
        e1.record()
        torch.cuda.synchronize()

        def over_ranks(x: float, op) -> float:
            t = torch.tensor([x], dtype=torch.float64, device=dev)
            if world.world_size > 1:
                dist.all_reduce(t, op=op)
            return float(t.item())

        ms = over_ranks(e0.elapsed_time(e1), dist.ReduceOp.MAX)
        n_sync = int(over_ranks(float(len(syncs)), dist.ReduceOp.MAX))
        sync_ms = over_ranks(statistics.mean(p.get("outer_sync", 0.0) for p in syncs) if syncs else 0.0, dist.ReduceOp.MAX)
        wait_ms = over_ranks(statistics.mean(p.get("outer_wait", 0.0) for p in syncs) if syncs else 0.0, dist.ReduceOp.MAX)
        curve = [[step, over_ranks(v, dist.ReduceOp.SUM) / n_last] for step, v in losses]
        if world.rank == 0:
            print(json.dumps({
                "H": H, "steps": a.steps, "world": f"{a.stages} stages x {world.world_size // a.stages} replicas",
                "tokens_per_s": a.batch * a.seq * a.steps / (ms / 1e3), "ms_per_step": ms / a.steps, "syncs": n_sync,
                "outer_sync_ms": sync_ms, "outer_wait_ms": wait_ms,
                "exposed_share": (sync_ms + wait_ms) * n_sync / ms, "loss": [[s, round(v, 4)] for s, v in curve]}), flush=True)
        tr.logger.close()
        del tr
        torch.cuda.empty_cache()
    world.barrier()
    world.destroy()


if __name__ == "__main__":
    main()
