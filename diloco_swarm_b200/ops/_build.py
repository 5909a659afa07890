"""In-tree builds of the native libraries.

``libdswarm_host.so`` (g++) holds the routing/plan generator and works without
CUDA.  ``libdswarm_cuda.so`` (nvcc, sm_100a only) holds every kernel and the
symmetric-memory runtime.  Both are plain C-ABI shared objects loaded with
ctypes, so they build in seconds and carry no torch headers.
"""
from __future__ import annotations

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


def build_cuda(force: bool = False, verbose: bool = False, jobs: int = 8) -> str:
    srcs = cuda_sources()
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    if not force and _newer(CUDA_LIB, srcs + hdrs):
        return CUDA_LIB
    nvcc = nvcc_path()
    objdir = os.path.join(PKG_DIR, "build")
    os.makedirs(objdir, exist_ok=True)
    procs, objs = [], []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s) + ".o")
        objs.append(o)
        if not force and _newer(o, [s] + hdrs):
            continue
        cmd = [nvcc] + NVCC_FLAGS + ["-Xptxas", "-v", "-c", s, "-o", o]
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
    tmp = CUDA_LIB + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp] + objs
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    subprocess.check_call(cmd)
    os.replace(tmp, CUDA_LIB)
    return CUDA_LIB


if __name__ == "__main__":
    build_host(force="--force" in sys.argv, verbose=True)
    build_cuda(force="--force" in sys.argv, verbose=True)
    print("built", HOST_LIB, CUDA_LIB)
