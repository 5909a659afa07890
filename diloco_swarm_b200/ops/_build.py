"""In-tree builds of the native libraries.

``libdswarm_host.so`` (g++) holds the routing/plan generator and works without
CUDA.  ``libdswarm_cuda.so`` (nvcc, sm_100a only) holds every kernel and the
symmetric-memory runtime.  Both are plain C-ABI shared objects loaded with
ctypes, so they build in seconds and carry no torch headers.
"""
from __future__ import annotations

import contextlib
import fcntl
import glob
import os
import shutil
import subprocess
import sys
from typing import List

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG_DIR, "csrc")
HOST_LIB = os.path.join(PKG_DIR, "libdswarm_host.so")
CUDA_LIB = os.path.join(PKG_DIR, "libdswarm_cuda.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
    "--expt-relaxed-constexpr",
]


def _newer(target: str, sources: List[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def host_sources() -> List[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cpp")))


def cuda_sources() -> List[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def build_host(force: bool = False, verbose: bool = False) -> str:
    srcs = host_sources()
    if not force and _newer(HOST_LIB, srcs + [os.path.join(CSRC, "dswarm_host.h"), os.path.join(CSRC, "coll_index.h")]):
        return HOST_LIB
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("g++ not found: cannot build libdswarm_host.so")
    tmp = HOST_LIB + f".tmp{os.getpid()}"
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-o", tmp] + srcs
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    subprocess.check_call(cmd)
    os.replace(tmp, HOST_LIB)
    return HOST_LIB


def nvcc_path() -> str:
    for c in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found: cannot build libdswarm_cuda.so")


# Debugging builds of the kernel library, each in its own file beside the shipped one:
#   trace   -DDSWARM_TRACE: the GEMM and attention kernels stamp %globaltimer at their phase boundaries into a
#           registered buffer (benchmarks/timelines.py); the shipped kernels carry no such code.
#   bounds  -DDSWARM_BOUNDS: every global access of the memory-bound kernels and the GEMM epilogue is checked
#           against the extents the launcher was given; a bad index sets status 4 and the access is skipped.
VARIANTS = {"": [], "trace": ["-DDSWARM_TRACE"], "bounds": ["-DDSWARM_BOUNDS"]}


def cuda_lib_path(variant: str = "") -> str:
    if variant not in VARIANTS:
        raise ValueError(f"unknown library variant {variant!r} (known: {sorted(VARIANTS)})")
    return CUDA_LIB if not variant else os.path.join(PKG_DIR, f"libdswarm_cuda_{variant}.so")


@contextlib.contextmanager
def _build_lock():
    """One builder at a time per checkout: ranks started together by torchrun would otherwise run
    nvcc into the same object files."""
    fd = os.open(os.path.join(PKG_DIR, ".build.lock"), os.O_CREAT | os.O_RDWR, 0o644)
    try:
        fcntl.flock(fd, fcntl.LOCK_EX)
        yield
    finally:
        fcntl.flock(fd, fcntl.LOCK_UN)
        os.close(fd)


def build_cuda(force: bool = False, verbose: bool = False, jobs: int = 8, variant: str = "") -> str:
    target = cuda_lib_path(variant)
    srcs = cuda_sources()
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    if not force and _newer(target, srcs + hdrs):
        return target
    with _build_lock():
        if not force and _newer(target, srcs + hdrs):       # another rank built it while this one waited
            return target
        return _build_cuda_locked(target, srcs, hdrs, force, verbose, jobs, variant)


def _build_cuda_locked(target: str, srcs: List[str], hdrs: List[str], force: bool, verbose: bool, jobs: int,
                       variant: str) -> str:
    nvcc = nvcc_path()
    objdir = os.path.join(PKG_DIR, "build" + (f"_{variant}" if variant else ""))
    os.makedirs(objdir, exist_ok=True)
    procs, objs = [], []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s) + ".o")
        objs.append(o)
        if not force and _newer(o, [s] + hdrs):
            continue
        cmd = [nvcc] + NVCC_FLAGS + VARIANTS[variant] + ["-Xptxas", "-v", "-c", s, "-o", o]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        log = open(o + ".log", "w")
        procs.append((s, subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT), log))
        while len([p for p in procs if p[1].poll() is None]) >= jobs:
            procs[0][1].wait()
    failed = []
    for s, p, log in procs:
        p.wait()
        log.close()
        if p.returncode != 0:
            failed.append(s)
    if failed:
        msgs = []
        for s in failed:
            o = os.path.join(objdir, os.path.basename(s) + ".o.log")
            msgs.append(open(o).read()[-4000:])
        raise RuntimeError("nvcc failed for " + ", ".join(failed) + "\n" + "\n".join(msgs))
    tmp = target + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp] + objs
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    subprocess.check_call(cmd)
    os.replace(tmp, target)
    return target


if __name__ == "__main__":
    build_host(force="--force" in sys.argv, verbose=True)
    built = [build_cuda(force="--force" in sys.argv, verbose=True)]
    for v in VARIANTS:
        if v and f"--{v}" in sys.argv:
            built.append(build_cuda(force="--force" in sys.argv, verbose=True, variant=v))
    print("built", HOST_LIB, *built)
