"""Headline benchmark: GPT-2 small DiLoCo-SWARM training tokens/s.

    python bench.py [--gpus N --steps K --warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (the one the reference's headline names): GPT-2 small (12 layers, d 768,
12 heads, vocab 50304, seq 1024), global batch 512 sequences, microbatch 16,
bf16 compute with fp32 master weights, AdamW inner, SGD-Nesterov outer
(lr 0.7, momentum 0.9), synthetic Zipf(1.0) token ids, random init.
Topology per N: 1 -> 1 stage x 1, 2 -> 2 x 1, 4 -> 2 x 2, 8 -> 2 x 4.
The global batch is fixed, so this is strong scaling.  The outer sync runs
once inside the timed region (H = min(50, K)).

After the two headline regions the same process runs a few steps of plain SWARM
(per-step fused gradient all-reduce instead of DiLoCo) on a second trainer and
reports its tokens/s and the exposed part of the gradient sync, and, outside any
timed region, checks the fused collectives against NCCL on buffers of the
stage's real size (``collective_check``; a mismatch makes the run fail).

Two timed regions of K steps each, both on the device with CUDA events between
a barrier + synchronize on both sides, max over ranks:
  value  batches already resident on the device;
  e2e    through ``Trainer.train_step`` with each step's batch in pinned host
         memory (copied host-to-device inside the step) and the loss read back.
One step touches several GB of weights and activations, far more than the
126 MB L2, so no explicit L2 flush is done between steps.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOPOLOGY = {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (2, 4)}
# The unmodified reference (gloo + host staging) on the same kind of B200 box, same config, tokens/s as measured by an
# earlier driver run of `bench.py --impl reference`; the reference publishes no throughput (so vs_baseline is null).
REFERENCE_TOKENS_PER_S = {1: 483165.0, 2: 136634.0, 4: 200694.0, 8: 300112.0}
SMI_QUERY = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="small")
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--micro-batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--cap", type=int, default=8, help="max_micro_batches (in-flight microbatches per rank)")
    ap.add_argument("--layer-split", default="balanced")
    ap.add_argument("--engine", default="b200", choices=["b200", "torch"],
                    help="b200 = the sm_100a kernels (the product); torch = this framework's autograd engine on "
                         "library ops (cuBLAS, SDPA, NCCL), a library twin of the same algorithm for comparison")
    ap.add_argument("--collective", default="fused")
    ap.add_argument("--routing", default="uniform", choices=["uniform", "balanced"])
    ap.add_argument("--no-outer", action="store_true", help="plain SWARM (per-step gradient all-reduce)")
    ap.add_argument("--stages", type=int, default=0, help="pipeline stages (default: 1 for one GPU, else 2)")
    ap.add_argument("--H", type=int, default=0, help="DiLoCo sync interval (default: min(50, steps))")
    ap.add_argument("--timeline-steps", type=int, default=0,
                    help="diagnosis: record every rank's forwards and backwards of this many timed steps into "
                         "<log-dir>/bench<pid>/timeline (utils/timeline.py); adds events to the timed region")
    ap.add_argument("--log-dir", default=os.path.join(tempfile.gettempdir(), "dswarm_bench"))
    ap.add_argument("--recv-prefetch", type=int, default=1, help="pipeline receives posted this many operations ahead")
    ap.add_argument("--p2p", default="auto", choices=["auto", "nccl", "copy"], help="pipeline transport")
    ap.add_argument("--swarm-steps", type=int, default=-1,
                    help="timed steps of the plain-SWARM side measurement (default min(steps, 8); 0 skips it)")
    ap.add_argument("--no-collective-check", action="store_true")
    ap.add_argument("--reserve-gb", type=float, default=0.0,
                    help="device memory handed to the caching allocator in one piece at start (train.reserve_memory_gb)")
    ap.add_argument("--lm-head-chunks", type=int, default=1,
                    help="slices of a microbatch's rows that the LM head and the cross-entropy run over")
    return ap.parse_args()


class ClockSampler:
    def __init__(self, enabled: bool):
        self.proc, self.path = None, None
        if not enabled:
            return
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={SMI_QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, windows=()) -> dict:
        """Summary of the samples whose timestamp falls inside one of ``windows`` (pairs of
        ``datetime``; all samples when empty): the sampler is started before the warm-up steps so
        that its own start-up is not inside a timed region."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                c = [x.strip() for x in line.split(",")]
                if len(c) < 10:
                    continue
                try:
                    ts = datetime.datetime.strptime(c[0], "%Y/%m/%d %H:%M:%S.%f")
                    c = c[1:]
                    clk, mx, pw = float(c[1]), float(c[2]), float(c[3])
                except ValueError:
                    continue
                if windows and not any(a <= ts <= b for a, b in windows):
                    continue
                smax.append(mx)
                power.append(pw)
                if pw > 300:                      # samples under load
                    sm.append(clk)
                for n, v in zip(names, c[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples_under_load": len(sm),
                "reasons": sorted(reasons)}


def build_config(args, S: int, no_outer=None, run_suffix: str = ""):
    from diloco_swarm_b200.config import Config, load_toml
    model = load_toml(os.path.join(ROOT, "configs", "model", f"gpt2-{args.model}.toml"))
    H = args.H if args.H > 0 else max(1, min(50, args.steps))
    no_outer = args.no_outer if no_outer is None else no_outer
    outer = {"type": "None", "lr": 0.0} if no_outer else {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True}
    return Config(
        model=model,
        data={"path": "synthetic:zipf", "seq_length": args.seq, "num_examples": args.batch * 2, "pin_memory": True},
        train={"micro_batch_size": args.micro_batch, "batch_size": args.batch, "max_steps": 10 ** 6,
               "max_micro_batches": args.cap, "step_timeout": 600, "lm_head_chunks": args.lm_head_chunks, "reserve_memory_gb": args.reserve_gb,
               "inner_optimizer": {"type": "AdamW", "lr": 6e-4},
               "outer_optimizer": outer,
               "scheduler": {"enable": True, "num_warmup_steps": 100, "type": "cosine"}},
        swarm={"num_stages": S, "sync_every_n_steps": 1 if no_outer else H, "layer_split": args.layer_split,
               "collective": args.collective, "routing": args.routing, "recv_prefetch": args.recv_prefetch,
               "p2p": args.p2p},
        eval={"enable": False}, sample={"enable": False},
        logging={"log_dir": args.log_dir,
                 "run_id": (f"bench{os.getpid()}" if args.timeline_steps == 0 else "bench") + run_suffix,
                 "console": {"log_level": "ERROR"}, "file": {"log_level": "ERROR"},
                 "timeline_steps": args.timeline_steps, "timeline_start": args.warmup + 1},
        engine=args.engine), H


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist
    from diloco_swarm_b200.ops import _lib
    from diloco_swarm_b200.train import Trainer
    from diloco_swarm_b200.utils import data as D

    N = args.gpus
    S, R = TOPOLOGY.get(N, (2 if N % 2 == 0 else 1, N // 2 if N % 2 == 0 else N))
    if args.stages > 0:
        S, R = args.stages, N // args.stages
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    if world_size != N:
        raise SystemExit(f"--gpus {N} needs {N} ranks (launch with torch.distributed.run); WORLD_SIZE={world_size}")
    cfg, H = build_config(args, S)
    tr = Trainer(cfg)
    tr.num_train_steps = 10 ** 6
    rank = tr.world.rank
    dev = tr.device

    tok = D.ByteTokenizer()
    ds = D.get_dataset(cfg.data, tok, seed=0)
    host = [{k: v.pin_memory() for k, v in D.collate(ds, i * args.batch, (i + 1) * args.batch).items()} for i in range(2)]
    resident = [{k: v.to(dev) for k, v in b.items()} for b in host]
    h2d = 0
    if tr.engine.is_first:
        h2d += host[0]["input_ids"].numel() * 8
    if tr.engine.is_last:
        h2d += (host[0]["target_ids"].numel() + host[0]["attention_mask"].numel()) * 8
    step_no = [0]

    active = [tr]
    sync_phases = []          # device phases of every step that synchronised, in order

    def one(batches):
        step_no[0] += 1
        t = active[0]
        before = t.last_sync_phase_ms
        local, _ = t.train_step(step_no[0], batches[step_no[0] % 2])
        if t.last_sync_phase_ms is not before:
            sync_phases.append(t.last_sync_phase_ms)
        return local

    windows, per_step, mallocs = [], [], []

    def timed(batches, steps):
        tr.world.barrier()
        torch.cuda.synchronize()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        l0 = _lib.launch_count()
        a0 = torch.cuda.memory_stats().get("num_device_alloc", 0)
        t0 = datetime.datetime.now()
        marks[0].record()
        last = None
        for i in range(steps):
            last = one(batches)
            marks[i + 1].record()
        torch.cuda.synchronize()
        windows.append((t0, datetime.datetime.now()))
        mallocs.append(torch.cuda.memory_stats().get("num_device_alloc", 0) - a0)
        per_step.append([marks[i].elapsed_time(marks[i + 1]) for i in range(steps)])
        ms = torch.tensor([marks[0].elapsed_time(marks[steps])], dtype=torch.float64, device=dev)
        tr.world.barrier()
        if world_size > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), _lib.launch_count() - l0, last

    sampler = ClockSampler(rank == 0)          # started ahead of the warm-up; only samples inside the timed windows count
    for _ in range(args.warmup):
        one(resident)
    ms_dev, launches, last = timed(resident, args.steps)
    for _ in range(1):
        one(host)
    ms_e2e, _, last_e2e = timed(host, args.steps)
    clocks = sampler.stop(windows) if rank == 0 else None
    tokens = args.batch * args.seq * args.steps
    # the loss lives on the last stage (rank 0 may be a first-stage rank); every last-stage replica reports the
    # sum over its own microbatches divided by M/R, so the mean over those replicas is the batch loss
    loss_t = torch.tensor([last.loss if (last and tr.engine.is_last) else 0.0], dtype=torch.float64, device=dev)
    if world_size > 1:
        dist.all_reduce(loss_t, op=dist.ReduceOp.SUM)
        loss_t /= len(tr.world.last_stage_ranks)
    # Device time of the outer sync (fused all-reduce + Nesterov + write-back + bf16 refresh of the weights) in the
    # steps that ran one, max over ranks, mean over those steps; the wait for the slowest replica before it is
    # reported separately.  Roofline: replica r reads its 1/R slice from R - 1 peers and writes it to R - 1
    # peers, 2 (R-1)/R 4n bytes per direction, over the slower of the two figures below.
    def max_over_ranks(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world_size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    n_sync = max_over_ranks(float(len(sync_phases)))
    outer_ms = max_over_ranks(statistics.mean(p.get("outer_sync", 0.0) for p in sync_phases) if sync_phases else 0.0)
    outer_wait_ms = max_over_ranks(statistics.mean(p.get("outer_wait", 0.0) for p in sync_phases) if sync_phases else 0.0)
    stage_elems = int(max_over_ranks(float(getattr(tr.engine, "n", 0))))
    outer_info = {"ms": outer_ms if n_sync else None, "wait_for_slowest_replica_ms": outer_wait_ms if n_sync else None,
                  "steps_with_a_sync": int(n_sync), "stage_elements": stage_elems, "replicas": R}
    if R > 1 and n_sync and outer_ms > 0:
        link_bytes = 2.0 * (R - 1) / R * 4.0 * stage_elems
        outer_info["nvlink_bytes_per_direction"] = link_bytes
        outer_info["includes"] = "fused kernel + bf16 refresh of the stage's weights (one pass over local memory)"
        outer_info["frac_of_770_GBs_measured_peer_copy"] = link_bytes / (outer_ms * 1e-3) / 770e9
        outer_info["frac_of_900_GBs_nominal"] = link_bytes / (outer_ms * 1e-3) / 900e9
    value = tokens / (ms_dev / 1e3)
    e2e = tokens / (ms_e2e / 1e3)

    # ---- plain SWARM in the same process: per-step fused gradient all-reduce, bucket-wise under the last backward
    swarm = None
    k2 = min(args.steps, 8) if args.swarm_steps < 0 else args.swarm_steps
    if k2 > 0 and not args.no_outer and args.timeline_steps == 0:
        cfg2, _ = build_config(args, S, no_outer=True, run_suffix="_swarm")
        tr2 = Trainer(cfg2, world=tr.world)
        tr2.num_train_steps = 10 ** 6
        active[0] = tr2
        first = len(sync_phases)
        for _ in range(3):
            one(resident)
        ms_sw, _, _ = timed(resident, k2)
        exposed = [p.get("grad_sync", 0.0) for p in sync_phases[first + 3:]]
        # The phase runs from the end of a rank's last backward to the end of its last bucket's all-reduce.  On the
        # replica that reaches its last backward last nobody is waited for, so its figure (the minimum over the
        # ranks) is what the synchronisation itself leaves exposed; on the others the phase is mostly the wait
        # for that replica (routing gives the replicas different loads), reported as the maximum.
        mine = statistics.mean(exposed) if exposed else 0.0
        t = torch.tensor([mine if R > 1 else 1e9], dtype=torch.float64, device=dev)
        if world_size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        swarm = {"swarm_tokens_per_s": args.batch * args.seq * k2 / (ms_sw / 1e3), "swarm_ms_per_step": ms_sw / k2,
                 "steps": k2, "warmup": 3,
                 "grad_sync_exposed_ms": float(t.item()) if R > 1 else 0.0,
                 "grad_sync_incl_wait_for_slowest_replica_ms": max_over_ranks(mine),
                 "grad_wire_dtype": cfg2.swarm.grad_wire_dtype}
        tr2.logger.close()
        active[0] = tr

    # ---- the fused collectives against NCCL on this box, outside the timed regions
    check = {"status": "skipped"}
    if not args.no_collective_check and args.engine == "b200" and args.collective in ("fused", "nvls"):
        from diloco_swarm_b200.parallel.collectives import check_against_nccl
        grp = tr.world.curr_stage_group if R > 1 else None
        check = check_against_nccl(grp, dev, tr.engine.n, tr.engine.buckets, multicast=args.collective == "nvls")
        bad = max_over_ranks(1.0 if check["status"] == "mismatch" else 0.0)
        if bad:
            check["status"] = "mismatch"
    out = {
        "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": N, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic Zipf(1.0) token ids, random-init weights",
        "impl": "ours",
        "config": {"model": f"gpt2-{args.model}", "global_batch": args.batch, "seq_len": args.seq,
                   "micro_batch": args.micro_batch, "parallelism": f"{S} stages x {R} replicas",
                   "algorithm": "swarm" if args.no_outer else f"diloco-swarm H={H}",
                   "max_micro_batches": args.cap, "layer_split": args.layer_split,
                   "layers_per_stage": tr.config.swarm.layer_split if S > 1 else str(tr.config.model.n_layer),
                   "engine": args.engine,
                   "collective": args.collective, "p2p": type(tr.comm).__name__,
                   "routing": args.routing, "allocator_pool_gb": args.reserve_gb, "lm_head_chunks": args.lm_head_chunks,
                   **({"timeline_steps": args.timeline_steps} if args.timeline_steps else {}),
                   "l2": "per-step working set (GBs) exceeds the 126 MB L2; no explicit flush"},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8},
        "gpu_launches": launches,
        "outer_sync": outer_info,
        "outer_sync_ms": outer_info["ms"],
        **(swarm or {}),
        "collective_check": check["status"], "collective_check_detail": check,
        # only for the configuration the reference arm was measured on (GPT-2 small, default batch and topology)
        "vs_reference_measured_earlier": (value / REFERENCE_TOKENS_PER_S[N])
        if (N in REFERENCE_TOKENS_PER_S and args.model == "small" and args.batch == 512 and args.micro_batch == 16
            and args.seq == 1024 and args.stages in (0, 1 if N == 1 else 2)) else None,
        "loss": float(loss_t.item()),
        "step_ms_rank0": {"device_resident_inputs": per_step[0], "e2e": per_step[1]},
        "cuda_mallocs_in_timed_regions_rank0": mallocs,
        "host_enqueue_ms_last_step": tr.last_enqueue_s * 1e3,
        "device_phases_ms_last_step_rank0": tr.last_phase_ms,
    }
    tr.world.barrier()
    tr.logger.close()
    tr.world.destroy()
    if check["status"] == "mismatch":
        if rank == 0:
            print(json.dumps(out), flush=True)
        raise SystemExit("collective_check failed: the fused collectives disagree with NCCL: " + json.dumps(check))
    return out if rank == 0 else {}


def main():
    args = parse_args()
    if args.impl == "reference":
        from baseline.run_reference import run_reference
        out = run_reference(args)
    else:
        out = run_ours(args)
    if out:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
