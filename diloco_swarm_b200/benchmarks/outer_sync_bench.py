"""Outer-sync and gradient all-reduce microbenchmark over a stage's replicas.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node R --master-addr 127.0.0.1 --master-port P \
        -m diloco_swarm_b200.benchmarks.outer_sync_bench [--sizes-mb 1,16,256,1024,3072] [--iters 5]

All R ranks form one stage (1 stage x R replicas).  For each message size
(fp32 elements, values N(0, 1e-3) from a seed) it times, on the device with CUDA
events, max over ranks:

  fused outer sync   one kernel: peer loads of every replica's weights, mean,
                     pseudo-gradient, Nesterov momentum, write-back to all replicas
  baseline           what the reference's algorithm costs with a library collective:
                     pseudo-gradient, NCCL all_reduce, divide, torch.optim.SGD(nesterov)
                     step on the global copy, copy back to the local weights
  fused grad sync    one kernel: sum over replicas, 1/R, write-back (fp32 and bf16 wire)
  NCCL grad sync     all_reduce + scale

Roofline: each GPU must receive (R-1)/R of the buffer once as peer loads and once
as peer stores, i.e. 2*(R-1)/R*4N bytes per direction, over the measured 770 GB/s
per direction (nominal 900).  ``frac`` = that time / measured time.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops._lib import Status, load_all_kernels
from ..parallel.collectives import GradSync, OuterSync
from ..parallel.symm import SymmetricBuffer

NVLINK_GBS = 770.0


def timed(fn, iters, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ms = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    t = torch.tensor([sorted(ms)[len(ms) // 2]], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", default="1,4,16,64,256,1024,3072")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--blocks", type=int, default=0)
    a = ap.parse_args()
    rank, R = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=R,
                            init_method=f"tcp://{os.environ['MASTER_ADDR']}:{os.environ['MASTER_PORT']}")
    group = dist.group.WORLD
    load_all_kernels()
    status = Status(dev)
    rows = []
    for mb in [float(x) for x in a.sizes_mb.split(",")]:
        n = int(mb * (1 << 20) / 4) // (8 * R) * (8 * R)
        nbytes = 4 * n
        g = torch.Generator(device="cuda").manual_seed(1234 + rank)
        theta = SymmetricBuffer(nbytes, dev, group)
        tview = theta.view(torch.float32, n)
        tview.normal_(0.0, 1e-3, generator=g)
        outer = OuterSync(theta, n, dev, 0.7, 0.9, True, group, status, blocks=a.blocks)
        # --- fused outer sync
        ms_fused = timed(outer.step, a.iters)
        # --- baseline: NCCL all-reduce + torch SGD (Nesterov) + copy back
        glob = torch.nn.Parameter(tview.clone())
        opt = torch.optim.SGD([glob], lr=0.7, momentum=0.9, nesterov=True)

        def baseline():
            glob.grad = glob.data - tview
            dist.all_reduce(glob.grad)
            glob.grad.div_(R)
            opt.step()
            tview.copy_(glob.data)
        ms_base = timed(baseline, a.iters)
        # --- gradient all-reduce
        del glob, opt
        grad = SymmetricBuffer(nbytes, dev, group)
        gview = grad.view(torch.float32, n)
        gview.normal_(0.0, 1e-3, generator=g)
        gs32 = GradSync(grad, n, dev, group, wire_bf16=False, status=status, blocks=a.blocks)
        ms_g32 = timed(gs32.all, a.iters)
        gs16 = GradSync(grad, n, dev, group, wire_bf16=True, status=status, blocks=a.blocks)
        ms_g16 = timed(gs16.all, a.iters)

        def nccl_grad():
            dist.all_reduce(gview)
            gview.mul_(1.0 / R)
        ms_gn = timed(nccl_grad, a.iters)
        status.raise_if_set()
        roof_ms = 2.0 * (R - 1) / R * nbytes / (NVLINK_GBS * 1e9) * 1e3 if R > 1 else float("nan")
        row = {"size_mb": mb, "n": n, "R": R, "outer_fused_ms": ms_fused, "outer_nccl_sgd_ms": ms_base,
               "grad_fused_f32_ms": ms_g32, "grad_fused_bf16_ms": ms_g16, "grad_nccl_ms": ms_gn,
               "roofline_ms": roof_ms, "outer_frac_of_nvlink_roofline": roof_ms / ms_fused if R > 1 else None,
               "grad_f32_frac_of_nvlink_roofline": roof_ms / ms_g32 if R > 1 else None,
               "outer_algbw_gbs": nbytes / ms_fused / 1e6, "speedup_vs_nccl_sgd": ms_base / ms_fused}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        torch.cuda.synchronize()
        dist.barrier()                      # nobody may still be reading a peer's buffer
        for b in (gs16.stage_buf, gs16.flags, gs32.flags, grad, outer.flags, theta):
            if b is not None:
                b.close()
        del outer, gs32, gs16, tview, gview
        torch.cuda.empty_cache()
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
