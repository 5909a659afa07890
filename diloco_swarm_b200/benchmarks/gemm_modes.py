"""Every GEMM of a GPT-2 training microbatch with the epilogue it runs with.

    python -m diloco_swarm_b200.benchmarks.gemm_modes --M 16384 --d 768 --V 50304 [--iters 20]

``kernel_cases --case gemm`` times the plain-store epilogue; inside a training
step most GEMMs carry fused work (bias, exact GELU with a second output,
residual add, multiply by the saved GELU derivative, fp32 accumulation into the main
gradient under split-K).  This tool times each call exactly as
``models/engine_b200.py`` issues it (same operand layouts, same tile choice,
same split) and, beside it, ``torch.matmul`` on the same operands: the library
GEMM alone, without the elementwise kernels a library path would add.  One
JSON line per GEMM plus a total.  CUDA events, operands L2-resident across
iterations unless ``--flush-l2``.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import kernels as K
from .kernel_cases import bf, timeit


def cases(M: int, d: int, V: int):
    x_d, x_3d, x_4d = bf(M, d), bf(M, 3 * d), bf(M, 4 * d)
    w_qkv, w_o, w_fc, w_pr, w_head = bf(3 * d, d), bf(d, d), bf(4 * d, d), bf(d, 4 * d), bf(V, d)
    b_3d, b_d, b_4d = (torch.randn(n, device="cuda") for n in (3 * d, d, 4 * d))
    h = bf(M, 4 * d)
    logits = bf(M, V) if V > 0 else None
    f32 = lambda m, n: torch.zeros(m, n, device="cuda")
    acc_qkv, acc_o, acc_fc, acc_pr = f32(3 * d, d), f32(d, d), f32(4 * d, d), f32(d, 4 * d)
    out = [
        ("qkv fwd (bias)", (M, 3 * d, d), lambda: K.gemm(x_d, w_qkv, bias=b_3d), lambda: x_d @ w_qkv.t()),
        ("out-proj fwd (bias+resid)", (M, d, d), lambda: K.gemm(x_d, w_o, mode=K.EPI_RESID, bias=b_d, resid=x_d),
         lambda: x_d @ w_o.t()),
        ("fc fwd (bias+gelu, gelu' saved)", (M, 4 * d, d),
         lambda: K.gemm(x_d, w_fc, mode=K.EPI_GELU, bias=b_4d, aux_out=h), lambda: x_d @ w_fc.t()),
        ("proj fwd (bias+resid)", (M, d, 4 * d), lambda: K.gemm(x_4d, w_pr, mode=K.EPI_RESID, bias=b_d, resid=x_d),
         lambda: x_4d @ w_pr.t()),
        ("proj dgrad (x saved gelu')", (M, 4 * d, d), lambda: K.gemm(x_d, w_pr, b_t=False, mode=K.EPI_MUL, aux_in=h),
         lambda: x_d @ w_pr),
        ("fc dgrad", (M, d, 4 * d), lambda: K.gemm(x_4d, w_fc, b_t=False), lambda: x_4d @ w_fc),
        ("out-proj dgrad", (M, d, d), lambda: K.gemm(x_d, w_o, b_t=False), lambda: x_d @ w_o),
        ("qkv dgrad", (M, d, 3 * d), lambda: K.gemm(x_3d, w_qkv, b_t=False), lambda: x_3d @ w_qkv),
        ("proj wgrad (split-K, fp32 +=)", (d, 4 * d, M),
         lambda: K.gemm(x_d, x_4d, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=acc_pr,
                        split_k=K.wgrad_split(d, 4 * d, M)), lambda: x_d.t() @ x_4d),
        ("fc wgrad", (4 * d, d, M),
         lambda: K.gemm(x_4d, x_d, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=acc_fc,
                        split_k=K.wgrad_split(4 * d, d, M)), lambda: x_4d.t() @ x_d),
        ("out-proj wgrad", (d, d, M),
         lambda: K.gemm(x_d, x_d, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=acc_o,
                        split_k=K.wgrad_split(d, d, M)), lambda: x_d.t() @ x_d),
        ("qkv wgrad", (3 * d, d, M),
         lambda: K.gemm(x_3d, x_d, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=acc_qkv,
                        split_k=K.wgrad_split(3 * d, d, M)), lambda: x_3d.t() @ x_d),
    ]
    per_block = len(out)
    if V > 0:
        acc_head = f32(V, d)
        out += [
            ("lm-head fwd", (M, V, d), lambda: K.gemm(x_d, w_head), lambda: x_d @ w_head.t()),
            ("lm-head dgrad", (M, d, V), lambda: K.gemm(logits, w_head, b_t=False), lambda: logits @ w_head),
            ("lm-head wgrad", (V, d, M),
             lambda: K.gemm(logits, x_d, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=acc_head,
                            split_k=K.wgrad_split(V, d, M)), lambda: logits.t() @ x_d),
        ]
    return out, per_block


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--d", type=int, default=768)
    ap.add_argument("--V", type=int, default=50304, help="0 leaves the LM head out")
    ap.add_argument("--layers", type=int, default=12, help="blocks counted in the per-microbatch total")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--flush-l2", action="store_true")
    ap.add_argument("--no-library", action="store_true")
    a = ap.parse_args()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if a.flush_l2 else None
    cs, per_block = cases(a.M, a.d, a.V)
    tot_ours = tot_lib = 0.0
    for i, (name, (m, n, k), ours, lib) in enumerate(cs):
        ms = timeit(ours, a.warmup, a.iters, flush)
        ms_lib = None if a.no_library else timeit(lib, a.warmup, a.iters, flush)
        fl = 2.0 * m * n * k
        weight = a.layers if i < per_block else 1
        tot_ours += weight * ms
        tot_lib += weight * (ms_lib or 0.0)
        print(json.dumps({"gemm": name, "shape_mnk": [m, n, k], "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
                          "library_ms": None if ms_lib is None else round(ms_lib, 4),
                          "library_tflops": None if ms_lib is None else round(fl / ms_lib / 1e9, 1)}), flush=True)
    print(json.dumps({"per_microbatch_ms": round(tot_ours, 3), "library_matmul_only_ms": round(tot_lib, 3),
                      "layers": a.layers}))


if __name__ == "__main__":
    main()
