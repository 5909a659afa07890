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

  NVLS variants      (``--nvls``) the same kernels with multimem.ld_reduce / multimem.st on
                     multicast-bound buffers: reduction and broadcast inside the NVSwitch

Roofline of the peer-load kernels: each GPU receives (R-1)/R of the buffer as peer loads
and sends (R-1)/R of it as peer stores (and serves / receives the same for its peers), i.e.
2*(R-1)/R*4N bytes per direction.  Of the NVLS kernels: every GPU sends all R slices of its
copy to the switch for reduction and its own reduced slice for the broadcast, and receives its
reduced slice and the R broadcast slices, i.e. (1 + 1/R)*4N bytes per direction: more than the
peer-load form at R = 2, 1.2x less at R = 4, 1.56x less at R = 8.  The link bandwidth in the
denominator is measured in the same run on the same GPUs (every rank copies 1 GiB to its ring
neighbour with the copy engines, all at once, so both directions of every GPU's links are
busy); fractions are printed against that and against the nominal 900 GB/s per direction.
``frac`` = roofline time / measured time.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops._lib import Status, check, cuda_lib, load_all_kernels, stream_ptr
from ..parallel.collectives import GradSync, OuterSync
from ..parallel.symm import SymmetricBuffer

NVLINK_NOMINAL_GBS = 900.0


def peer_copy_gbs(group, dev, rank: int, R: int, nbytes: int = 1 << 30, iters: int = 5) -> dict:
    """Per-direction NVLink bandwidth with every GPU sending to and receiving from a ring neighbour at once:
    by the copy engines (cudaMemcpyAsync) and by SM stores (an elementwise copy kernel writing peer memory)."""
    from ..parallel.symm import _CudaArray
    buf = SymmetricBuffer(nbytes, dev, group)
    src = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    dst = buf.peer_ptrs[(rank + 1) % R]
    lib = cuda_lib()
    ms_ce = timed(lambda: check(lib.dsw_copy_async(dst, src.data_ptr(), nbytes, stream_ptr()), "copy"), iters)
    peer_view = torch.as_tensor(_CudaArray(dst, nbytes, buf), device=dev).view(torch.float32)
    src32 = src.view(torch.float32)
    ms_sm = timed(lambda: peer_view.copy_(src32), iters)
    torch.cuda.synchronize()
    dist.barrier()
    del peer_view
    buf.close()
    return {"copy_engine": nbytes / ms_ce / 1e6, "sm_stores": nbytes / ms_sm / 1e6}


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
    ap.add_argument("--nvls", action="store_true", help="also time the multimem variants (multicast-bound buffers)")
    a = ap.parse_args()
    rank, R = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=R,
                            init_method=f"tcp://{os.environ['MASTER_ADDR']}:{os.environ['MASTER_PORT']}")
    group = dist.group.WORLD
    load_all_kernels()
    status = Status(dev)
    links = peer_copy_gbs(group, dev, rank, R) if R > 1 else {"copy_engine": float("nan"), "sm_stores": float("nan")}
    link_gbs = max(links.values())
    if rank == 0:
        print(json.dumps({"peer_copy_gbs_per_direction_measured": links, "roofline_uses": link_gbs,
                          "nominal_gbs": NVLINK_NOMINAL_GBS, "R": R}), flush=True)
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
        p2p_bytes = 2.0 * (R - 1) / R * nbytes
        roof_ms = p2p_bytes / (link_gbs * 1e9) * 1e3 if R > 1 else float("nan")
        roof_nominal_ms = p2p_bytes / (NVLINK_NOMINAL_GBS * 1e9) * 1e3 if R > 1 else float("nan")
        row = {"size_mb": mb, "n": n, "R": R, "outer_fused_ms": ms_fused, "outer_nccl_sgd_ms": ms_base,
               "grad_fused_f32_ms": ms_g32, "grad_fused_bf16_ms": ms_g16, "grad_nccl_ms": ms_gn,
               "p2p_bytes_per_direction": p2p_bytes, "roofline_ms_measured_link": roof_ms,
               "outer_frac_of_measured_link": roof_ms / ms_fused if R > 1 else None,
               "outer_frac_of_nominal_900": roof_nominal_ms / ms_fused if R > 1 else None,
               "grad_f32_frac_of_measured_link": roof_ms / ms_g32 if R > 1 else None,
               "grad_f32_frac_of_nominal_900": roof_nominal_ms / ms_g32 if R > 1 else None,
               "outer_algbw_gbs": nbytes / ms_fused / 1e6, "speedup_vs_nccl_sgd": ms_base / ms_fused}
        nv_bufs = []
        if a.nvls and R > 1:
            th2 = SymmetricBuffer(nbytes, dev, group, multicast=True)
            nv_bufs.append(th2)
            if th2.mc_ptr:
                th2.view(torch.float32, n).normal_(0.0, 1e-3, generator=g)
                outer2 = OuterSync(th2, n, dev, 0.7, 0.9, True, group, status, blocks=a.blocks)
                ms_o2 = timed(outer2.step, a.iters)
                gr2 = SymmetricBuffer(nbytes, dev, group, multicast=True)
                gr2.view(torch.float32, n).normal_(0.0, 1e-3, generator=g)
                g2_32 = GradSync(gr2, n, dev, group, wire_bf16=False, status=status, blocks=a.blocks)
                ms_g2_32 = timed(g2_32.all, a.iters)
                g2_16 = GradSync(gr2, n, dev, group, wire_bf16=True, status=status, blocks=a.blocks)
                ms_g2_16 = timed(g2_16.all, a.iters)
                status.raise_if_set()
                nv_bytes = (1.0 + 1.0 / R) * nbytes
                row.update(outer_nvls_ms=ms_o2, grad_nvls_f32_ms=ms_g2_32, grad_nvls_bf16_ms=ms_g2_16,
                           nvls_bytes_per_direction=nv_bytes,
                           outer_nvls_frac_of_measured_link=nv_bytes / (link_gbs * 1e9) * 1e3 / ms_o2,
                           outer_nvls_frac_of_nominal_900=nv_bytes / (NVLINK_NOMINAL_GBS * 1e9) * 1e3 / ms_o2)
                nv_bufs += [g2_16.stage_buf, g2_16.flags, g2_32.flags, gr2, outer2.flags]
            else:
                row["nvls"] = "no multicast address on this box"
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        torch.cuda.synchronize()
        dist.barrier()                      # nobody may still be reading a peer's buffer
        for b in [gs16.stage_buf, gs16.flags, gs32.flags, grad, outer.flags, theta] + nv_bufs[::-1]:
            if b is not None:
                b.close()
        del outer, gs32, gs16, tview, gview
        torch.cuda.empty_cache()
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
