"""The ctypes bindings against the C headers of the two native libraries.

The Python layer calls the libraries through ctypes, where a wrong argument
list is not an error but a garbage call.  The headers are compiled into every
source file (a definition that differs from its declaration does not build),
so comparing the bindings with the headers ties all three together.  Also
checks that the built libraries export what the headers declare.  No GPU.
"""
import ctypes
import os
import re

import pytest

from diloco_swarm_b200.ops import _build, _lib
from diloco_swarm_b200.parallel import schedule

CSRC = _build.CSRC


def _ctype(param: str):
    """ctypes class that carries a C parameter written as in the headers."""
    p = param.strip()
    if "*" in p or p.startswith("cudaStream_t"):
        return ctypes.c_void_p
    words = p.split()[:-1]                      # drop the parameter name
    t = " ".join(w for w in words if w != "const")
    return {"int": ctypes.c_int, "long long": ctypes.c_longlong, "float": ctypes.c_float,
            "unsigned": ctypes.c_uint, "size_t": ctypes.c_size_t, "uint64_t": ctypes.c_uint64,
            "double": ctypes.c_double}[t]


def _declarations(header: str):
    text = open(os.path.join(CSRC, header)).read()
    text = re.sub(r"//[^\n]*", "", text)
    out = {}
    for name, params in re.findall(r"\bint\s+(dsw_\w+)\s*\(([^)]*)\)\s*;", text):
        params = params.strip()
        out[name] = [] if params in ("", "void") else [_ctype(p) for p in params.split(",")]
    return out


def _same(a, b) -> bool:
    # a pointer may be bound as c_void_p or as POINTER(c_void_p): both travel as one machine word
    is_ptr = lambda t: t is ctypes.c_void_p or hasattr(t, "contents") or issubclass(t, ctypes._Pointer)
    return a is b or (is_ptr(a) and is_ptr(b))


def test_cuda_bindings_match_the_header():
    decl = {**_declarations("dswarm.h"), **_declarations("dswarm_noalloc.h")}
    assert len(decl) >= 35
    for name, argtypes in _lib._SIGS.items():
        assert name in decl, f"{name} is bound in ops/_lib.py but not declared in dswarm.h"
        want = decl[name]
        assert len(argtypes) == len(want), f"{name}: {len(argtypes)} bound arguments, {len(want)} declared"
        for i, (a, b) in enumerate(zip(argtypes, want)):
            assert _same(a, b), f"{name}: argument {i} bound as {a.__name__}, declared as {b.__name__}"


def test_host_bindings_match_the_header():
    decl = _declarations("dswarm_host.h")
    lib = schedule._host()
    assert set(decl) == {"dsw_route", "dsw_route_weighted", "dsw_plan", "dsw_coll_touch_map"}
    for name, want in decl.items():
        got = list(getattr(lib, name).argtypes)
        assert len(got) == len(want), name
        for i, (a, b) in enumerate(zip(got, want)):
            assert _same(a, b), f"{name}: argument {i} bound as {a.__name__}, declared as {b.__name__}"
    assert (schedule.FWD, schedule.BWD, schedule.FWD_BWD) == (0, 1, 2)


def test_every_definition_is_declared():
    """An exported function that is missing from the headers would escape the checks above."""
    decl = {**_declarations("dswarm.h"), **_declarations("dswarm_noalloc.h"), **_declarations("dswarm_host.h")}
    defined = set()
    for src in _build.cuda_sources() + _build.host_sources():
        text = open(src).read()
        defined |= set(re.findall(r'extern "C" int (dsw_\w+)\s*\(', text))
        defined |= set(re.findall(r"^DSW_BOUNDS_TU\((dsw_\w+)\)", text, flags=re.M))     # macro-made readers
        for block in re.findall(r'extern "C" \{(.*?)\n\}  // extern "C"', text, flags=re.S):
            defined |= set(re.findall(r"^int (dsw_\w+)\s*\(", block, flags=re.M))
    assert defined == set(decl), (sorted(defined - set(decl)), sorted(set(decl) - defined))


def test_built_libraries_export_the_declared_symbols():
    cuda = ctypes.CDLL(_build.build_cuda())      # nvcc cross-compiles without a GPU
    for name in {**_declarations("dswarm.h"), **_declarations("dswarm_noalloc.h")}:
        assert hasattr(cuda, name), f"{name} is declared but not exported by libdswarm_cuda.so"
    host = ctypes.CDLL(_build.build_host())
    for name in _declarations("dswarm_host.h"):
        assert hasattr(host, name), name
    assert cuda.dsw_max_peers() == 8 and cuda.dsw_layernorm_bwd_blocks(16384) <= 296


def test_wrappers_run_against_a_stub_of_the_header():
    """benchmarks/host_overhead.py: a no-op twin of the library generated from dswarm.h takes every call
    the wrappers make (argument counts and kinds fit), and the loader is put back afterwards."""
    from diloco_swarm_b200.benchmarks import host_overhead as H
    before = _lib._cuda
    res = H.measure(iters=20, M=512, d=256)
    assert _lib._cuda is before
    assert set(res) >= {"gemm forward (bias)", "adamw step"} and all(0 < v < 1e5 for v in res.values())
