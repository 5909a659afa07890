"""Single-kernel cases: timing with CUDA events and roofline fractions.

    python -m diloco_swarm_b200.benchmarks.kernel_cases --case gemm --M 16384 --N 2304 --K 768 --bn 256
    python -m diloco_swarm_b200.benchmarks.kernel_cases --case outer_sync --n 81000000 --R 4

Each case runs ``--warmup`` untimed launches, then ``--iters`` timed ones
between CUDA events, and prints one JSON line with the achieved rate and its
fraction of the measured peak (``MEASURED_PEAKS.json`` at the repository root
if present, else the stated fallbacks).  The same commands, with small sizes
and few iterations, are what the ncu summaries under ``profiles/`` were
captured from.  Collective cases emulate R replicas on one GPU with sequential
launches and barriers off (kernels that wait on each other never share a GPU),
so they measure the kernel's arithmetic and local memory traffic, not NVLink.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import kernels as K
from ..ops._lib import check, cuda_lib, stream_ptr
from ..parallel.collectives import shard_size
from ..parallel.symm import LocalPeerSet

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def timeit(fn, warmup, iters, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()                       # write a buffer larger than L2 between iterations
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def bf(*shape, scale=0.1):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True,
                    choices=["gemm", "layernorm_fwd", "layernorm_bwd", "cross_entropy", "adamw", "outer_sync",
                             "grad_allreduce", "attention"])
    ap.add_argument("--B", type=int, default=16)
    ap.add_argument("--T", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=2304)
    ap.add_argument("--K", type=int, default=768)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--variant", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--split", type=int, default=1)
    ap.add_argument("--library", action="store_true", help="gemm: time torch.matmul instead of the tcgen05 kernel")
    ap.add_argument("--n", type=int, default=81_000_000)
    ap.add_argument("--R", type=int, default=4)
    ap.add_argument("--bf16-wire", action="store_true")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--flush-l2", action="store_true")
    a = ap.parse_args()
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if a.flush_l2 else None
    out = {"case": a.case, "peaks": pk["source"]}
    if a.case == "gemm":
        M, N, Kd = a.M, a.N, a.K
        # --library times torch.matmul (cuBLAS) on the same operands: the comparison column of the profiles
        if a.variant == "nt":
            x, w = bf(M, Kd), bf(N, Kd)
            fn = (lambda: x @ w.t()) if a.library else (lambda: K.gemm(x, w, bn=a.bn))
        elif a.variant == "nn":
            x, w = bf(M, Kd), bf(Kd, N)
            fn = (lambda: x @ w) if a.library else (lambda: K.gemm(x, w, b_t=False, bn=a.bn))
        else:
            x, w = bf(Kd, M), bf(Kd, N)
            acc = torch.zeros(M, N, device="cuda")
            fn = (lambda: x.t() @ w) if a.library else (
                lambda: K.gemm(x, w, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=acc, split_k=a.split, bn=a.bn))
        ms = timeit(fn, a.warmup, a.iters, flush)
        tf = 2.0 * M * N * Kd / ms / 1e9
        out.update(shape=[M, N, Kd], variant=a.variant, bn=a.bn, library=bool(a.library), ms=ms, tflops=tf,
                   frac_of_peak=tf / pk["bf16_tflops"])
    elif a.case in ("layernorm_fwd", "layernorm_bwd"):
        M, d = a.M, a.K
        x, g, b = bf(M, d, scale=1.0), torch.randn(d, device="cuda"), torch.randn(d, device="cuda")
        y, mean, rstd = K.layernorm_fwd(x, g, b)
        if a.case == "layernorm_fwd":
            fn, nbytes = (lambda: K.layernorm_fwd(x, g, b)), 2 * M * d * 2
        else:
            dy, dres = bf(M, d), bf(M, d)
            dg, db, ds = (torch.zeros(d, device="cuda") for _ in range(3))
            fn = lambda: K.layernorm_bwd(dy, x, g, mean, rstd, dg, db, dres=dres, dres_sum=ds)
            nbytes = 4 * M * d * 2
        ms = timeit(fn, a.warmup, a.iters, flush)
        out.update(shape=[M, d], ms=ms, gbs=nbytes / ms / 1e6, frac_of_peak=nbytes / ms / 1e6 / pk["hbm_gbs"])
    elif a.case == "cross_entropy":
        M, V = a.M, a.N
        logits = bf(M, V, scale=2.0)
        tg = torch.randint(0, V, (M,), device="cuda")
        mask = torch.ones(M, dtype=torch.long, device="cuda")
        loss, cnt = torch.zeros((), device="cuda"), torch.zeros(1, device="cuda")
        fn = lambda: K.cross_entropy(logits, tg, mask, 1.0, loss, cnt, write_grad=True)
        ms = timeit(fn, a.warmup, a.iters, flush)
        nbytes = 2 * M * V * 2          # algorithmic: read the logits once, write the gradient once
        out.update(shape=[M, V], ms=ms, gbs=nbytes / ms / 1e6, frac_of_peak=nbytes / ms / 1e6 / pk["hbm_gbs"])
    elif a.case == "attention":
        from ..ops.attention import attention_bwd, attention_fwd
        B, T, nh = a.B, a.T, a.heads
        qkv = bf(B * T, 3 * nh * 64, scale=1.0)
        dout = bf(B * T, nh * 64, scale=1.0)
        _, ctx = attention_fwd(qkv, B, T, nh)
        ms_f = timeit(lambda: attention_fwd(qkv, B, T, nh), a.warmup, a.iters, flush)
        if ctx.native:
            ms_b = timeit(lambda: attention_bwd(dout, ctx), a.warmup, a.iters, flush)
        else:
            # the library path goes through autograd, whose graph serves one backward: time forward + backward
            # pairs and take the forward off
            ms_b = timeit(lambda: attention_bwd(dout, attention_fwd(qkv, B, T, nh)[1]), a.warmup, a.iters, flush) - ms_f
        fl = 4.0 * B * nh * T * T * 64 / 2          # causal: half of the score matrix
        out.update(shape=[B, T, nh, 64], native=bool(ctx.native), fwd_ms=ms_f, bwd_ms=ms_b,
                   fwd_tflops=fl / ms_f / 1e9, bwd_tflops=2.5 * fl / ms_b / 1e9,
                   fwd_frac_of_peak=fl / ms_f / 1e9 / pk["bf16_tflops"])
    elif a.case == "adamw":
        n = a.n // 8 * 8
        p, g, m, v = (torch.randn(n, device="cuda") * 0.01 for _ in range(4))
        v.abs_()
        p16 = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        stats = torch.ones(4, device="cuda")
        fn = lambda: K.adamw_step(p, g, m, v, p16, 1e-4, (0.9, 0.95), 1e-8, 0.1, 10, stats, zero_grad=True)
        ms = timeit(fn, a.warmup, a.iters, flush)
        nbytes = n * (4 * 4 + 4 * 4 + 2)   # read p,g,m,v; write p,g,m,v and the bf16 copy
        out.update(n=n, ms=ms, gbs=nbytes / ms / 1e6, frac_of_peak=nbytes / ms / 1e6 / pk["hbm_gbs"])
    else:
        R = a.R
        n = a.n // (8 * R) * (8 * R)
        bufs = [torch.randn(n, device="cuda") * 1e-3 for _ in range(R)]
        lib = cuda_lib()
        if a.case == "outer_sync":
            shard = shard_size(n, R, 4)
            tg = [torch.zeros(shard, device="cuda") for _ in range(R)]
            mom = [torch.zeros(shard, device="cuda") for _ in range(R)]
            peers = LocalPeerSet(bufs)

            def fn():
                for r in range(R):
                    check(lib.dsw_outer_sync(peers.table, None, tg[r].data_ptr(), mom[r].data_ptr(), n, shard, r, R, 0.7,
                                             0.9, 1, 1, 0, 0, 0, None, stream_ptr()), "outer")
            nbytes = n * 4 * (2 * R + 4.0) / 1.0      # all R launches: R reads + R writes of every slice, 4 shard passes
        else:
            shard = shard_size(n, R, 8)
            wire = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(R)] if a.bf16_wire else bufs
            peers = LocalPeerSet(wire)

            def fn():
                for phase in ((1, 2, 4) if a.bf16_wire else (7,)):
                    for r in range(R):
                        check(lib.dsw_grad_allreduce(peers.table, None, bufs[r].data_ptr(), 0, n, shard, r, R,
                                                     1 if a.bf16_wire else 0, 1, 0, 0, phase, 0, None, stream_ptr()), "grad")
            nbytes = n * 4 * 2 * R
        ms = timeit(fn, a.warmup, a.iters, flush)
        out.update(n=n, R=R, ms_all_replicas=ms, ms_per_replica=ms / R, local_gbs=nbytes / ms / 1e6,
                   note="replicas emulated on one GPU by sequential launches; NVLink is not exercised")
    print(json.dumps(out))


if __name__ == "__main__":
    main()
