"""Host time of a kernel launch through the Python entry points, measured without a GPU.

    python -m diloco_swarm_b200.benchmarks.host_overhead [--iters 2000]

A training step queues thousands of launches from one Python thread, so the time the host spends per
launch (argument checks, tile choice, pointer extraction, the ctypes call) decides how far ahead of the
device it can run.  This tool builds a twin of the kernel library in which every entry point of
``csrc/dswarm.h`` returns at once (generated from the header, compiled with the C compiler), binds the
package's wrappers to it, and times them on CPU tensors of the training shapes.  What it leaves out is
the driver's own launch cost and the caching allocator of the device.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import re
import shutil
import subprocess
import tempfile
import time
from typing import Callable, Dict

import torch

from ..ops import _build, _lib
from ..ops import kernels as K


def build_stub(out_dir: str) -> str:
    """A shared object that exports every function declared in dswarm.h as ``return 0``."""
    header = open(os.path.join(_build.CSRC, "dswarm.h")).read()
    header = re.sub(r"//[^\n]*", "", header)
    lines = ["#include <stddef.h>", "typedef void* cudaStream_t;"]
    for name, params in re.findall(r"\bint\s+(dsw_\w+)\s*\(([^)]*)\)\s*;", header):
        lines.append(f"int {name}({params}) {{ return 0; }}")
    src = os.path.join(out_dir, "dswarm_stub.c")
    with open(src, "w") as f:
        f.write("\n".join(lines) + "\n")
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        raise RuntimeError("a C compiler is needed to build the stub library")
    lib = os.path.join(out_dir, "libdswarm_stub.so")
    subprocess.check_call([cc, "-O2", "-shared", "-fPIC", "-o", lib, src])
    return lib


class StubLibrary:
    """Binds ops/_lib.py to the stub for the duration of a ``with`` block."""

    def __init__(self):
        self._dir = tempfile.mkdtemp(prefix="dswarm_stub_")
        self.lib = ctypes.CDLL(build_stub(self._dir))
        for name, argtypes in _lib._SIGS.items():
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = ctypes.c_int, argtypes

    def __enter__(self):
        self._saved = (_lib._cuda, _lib.stream_ptr, K.stream_ptr)
        _lib._cuda = self.lib
        _lib.stream_ptr = K.stream_ptr = lambda stream=None: 0
        return self

    def __exit__(self, *exc):
        _lib._cuda, _lib.stream_ptr, K.stream_ptr = self._saved
        shutil.rmtree(self._dir, ignore_errors=True)


def _time_us(fn: Callable[[], object], iters: int) -> float:
    fn()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t0) / iters * 1e6


def measure(iters: int = 2000, M: int = 16384, d: int = 768) -> Dict[str, float]:
    """Microseconds of host time per call of the main wrappers (outputs preallocated where the wrapper
    allows it, so that the CPU allocator does not stand in for the device's)."""
    bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16)
    with StubLibrary():
        x, w, bias, out = bf(M, d), bf(3 * d, d), torch.empty(3 * d), bf(M, 3 * d)
        dy, dw = bf(M, 3 * d), torch.empty(3 * d, d)
        gamma, beta = torch.empty(d), torch.empty(d)
        p, p16 = torch.empty(1 << 20), bf(1 << 20)
        stats = torch.zeros(4)
        res = {
            "gemm forward (bias)": _time_us(lambda: K.gemm(x, w, bias=bias, out=out), iters),
            "gemm weight gradient (split-K)": _time_us(
                lambda: K.gemm(dy, x, a_t=True, b_t=False, mode=K.EPI_ATOMIC_F32, out=dw,
                               split_k=K.wgrad_split(3 * d, d, M)), iters),
            "tile and split choice": _time_us(lambda: (K._pick_bn(M, 3 * d, 1), K.wgrad_split(3 * d, d, M)), iters),
            "layernorm forward (allocates 3 outputs)": _time_us(lambda: K.layernorm_fwd(x, gamma, beta), max(1, iters // 10)),
            "adamw step": _time_us(lambda: K.adamw_step(p, p, p, p, p16, 1e-3, (0.9, 0.95), 1e-8, 0.1, 1, stats), max(1, iters // 10)),
        }
    return res


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--iters", type=int, default=2000)
    a = ap.parse_args()
    print(json.dumps({k: round(v, 2) for k, v in measure(a.iters).items()}, indent=1))


if __name__ == "__main__":
    main()
