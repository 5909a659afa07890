"""In-kernel timelines of the GEMM and attention kernels.

    python -m diloco_swarm_b200.benchmarks.timelines --kernel gemm --M 16384 --N 2304 --K 768
    python -m diloco_swarm_b200.benchmarks.timelines --kernel attention --B 16 --T 1024 --heads 12

The kernels can stamp ``%globaltimer`` at their phase boundaries into a small
device buffer (``dsw_gemm_set_trace`` / ``dsw_attention_set_trace``; CTA 0 only,
32 ns resolution, off unless a buffer is registered).  This prints the
per-phase durations: for the GEMM the MMA-issuing thread's wait / issue / commit
per k-block, for attention the softmax (or row) warp 0 and the MMA thread per
tile.  It is a tuning aid; the stamps perturb the kernel slightly, so these are
not benchmark numbers.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import statistics

# the stamps are compiled into the tracing build of the library only (ops/_build.py: variant "trace")
os.environ.setdefault("DSWARM_LIB_VARIANT", "trace")

import torch

from ..ops import kernels as K
from ..ops._lib import cuda_lib
from ..ops.attention import attention_bwd, attention_fwd


def _bf(*shape, scale=0.1):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _setter(name):
    fn = getattr(cuda_lib(), name)
    fn.argtypes = [ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def gemm_timeline(M, N, Kd, bn=256, mode="store"):
    set_trace = _setter("dsw_gemm_set_trace")
    a, b = _bf(M, Kd), _bf(N, Kd)
    bias = torch.randn(N, device="cuda")
    extra = _bf(M, N)
    call = {"store": lambda: K.gemm(a, b, bn=bn),
            "bias": lambda: K.gemm(a, b, bn=bn, bias=bias),
            "gelu": lambda: K.gemm(a, b, bn=bn, bias=bias, mode=K.EPI_GELU, aux_out=extra),
            "resid": lambda: K.gemm(a, b, bn=bn, bias=bias, mode=K.EPI_RESID, resid=extra),
            "mul": lambda: K.gemm(a, b, bn=bn, mode=K.EPI_MUL, aux_in=extra)}[mode]
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    tr = torch.zeros(512, dtype=torch.int64, device="cuda")
    set_trace(tr.data_ptr())
    call()
    torch.cuda.synchronize()
    set_trace(None)
    raw = tr.cpu().tolist()
    t = [x for x in raw[:256] if x]
    waits = [t[i + 1] - t[i] for i in range(0, len(t) - 3, 4)]
    mmas = [t[i + 2] - t[i + 1] for i in range(0, len(t) - 3, 4)]
    commits = [t[i + 3] - t[i + 2] for i in range(0, len(t) - 3, 4)]
    period = [t[i + 4] - t[i] for i in range(0, len(t) - 4, 4)]
    kind = "CTA-pair kernel, 2 k-blocks per barrier" if bn == 512 else f"one-CTA kernel, bn={bn}"
    n_mma = 8 if bn == 512 else 4
    print(f"gemm {M}x{N}x{Kd} {mode} ({kind}): {len(waits)} barrier periods of CTA 0")
    for name, v in (("full-barrier wait", waits), (f"{n_mma} x tcgen05.mma", mmas), ("tcgen05.commit", commits),
                    ("period", period)):
        print(f"  {name:18s} median {statistics.median(v):6.0f} ns   mean {statistics.mean(v):7.1f} ns   max {max(v)} ns")
    print("  first periods:", period[:28])
    # CTA-pair kernel: the first epilogue warp's stamps per tile (start of the wait for the accumulator, got
    # it, tile written out)
    e = [x for x in raw[256:] if x]
    if len(e) >= 3:
        t0 = e[0]
        tiles = [(e[i] - t0, e[i + 1] - e[i], e[i + 2] - e[i + 1]) for i in range(0, len(e) - 2, 3)]
        print("  epilogue warp, per tile (start ns, wait for accumulator ns, drain + write-out ns):")
        print("   ", tiles[:16])
        print(f"  drain median {statistics.median(x[2] for x in tiles):.0f} ns, accumulator wait median "
              f"{statistics.median(x[1] for x in tiles):.0f} ns, tiles {len(tiles)}, span {e[-1] - t0} ns")


def attention_timeline(B, T, nh):
    set_trace = _setter("dsw_attention_set_trace")
    qkv, dout = _bf(B * T, 3 * nh * 64, scale=1.0), _bf(B * T, nh * 64, scale=1.0)
    for _ in range(3):
        _, ctx = attention_fwd(qkv, B, T, nh)
        attention_bwd(dout, ctx)
    torch.cuda.synchronize()
    tr = torch.zeros(512, dtype=torch.int64, device="cuda")

    def show(title, row_labels, mma_labels, row_first=None, mma_prefix=(), steps=5):
        """Stamps of one CTA, labelled: ``row_first`` names the (shorter) first step of the row warp."""
        t = tr.cpu().tolist()
        row, mma = [x for x in t[:256] if x], [x for x in t[256:] if x]
        t0 = min(row + mma)
        rnames = list(row_first or row_labels) + [row_labels[i % len(row_labels)] for i in range(len(row_labels) * (steps - 1))]
        mnames = list(mma_prefix) + [mma_labels[i % len(mma_labels)] for i in range(len(mma_labels) * steps)]
        print(title)
        print("  row warp 0 :", " ".join(f"{n}={x - t0}" for n, x in zip(rnames, row)))
        print("  MMA thread :", " ".join(f"{n}={x - t0}" for n, x in zip(mnames, mma)))
        print(f"  CTA span {max(row + mma) - t0} ns")

    set_trace(tr.data_ptr())
    _, ctx = attention_fwd(qkv, B, T, nh)
    torch.cuda.synchronize()
    show("attention forward, CTA (0,0) (last query tile: all kv tiles), ns since first stamp",
         ["waitS", "gotS", "max", "O_ready", "P_written"], ["S_issued", "P_ready", "PV_issued"])
    tr.zero_()
    attention_bwd(dout, ctx)
    torch.cuda.synchronize()
    # Row warp, per step: start, S and dP ready, P and dS in registers (S and dP released), P and dS written; from
    # the second step on, the dQ of the step before follows: its product done, staging tile free, staged.
    # MMA thread, per step: the next step's S/dP pair issued, P and dS ready, dV/dK/dQ issued.
    show("attention backward, CTA (0,0) (kv tile 0: all query tiles), ns since first stamp",
         ["start", "S_dP_ready", "in_regs", "written", "dQ_done", "stage_free", "staged"],
         ["next_S_dP_issued", "P_dS_ready", "dV_dK_dQ_issued"],
         row_first=["start", "S_dP_ready", "in_regs", "written"], mma_prefix=["S_dP_issued"])
    set_trace(None)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True, choices=["gemm", "attention"])
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=2304)
    ap.add_argument("--K", type=int, default=768)
    ap.add_argument("--bn", type=int, default=256, choices=[128, 256, 512], help="512 = the CTA-pair kernel")
    ap.add_argument("--mode", default="store", choices=["store", "bias", "gelu", "resid", "mul"], help="GEMM epilogue")
    ap.add_argument("--B", type=int, default=16)
    ap.add_argument("--T", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=12)
    a = ap.parse_args()
    if a.kernel == "gemm":
        gemm_timeline(a.M, a.N, a.K, a.bn, a.mode)
    else:
        attention_timeline(a.B, a.T, a.heads)


if __name__ == "__main__":
    main()
