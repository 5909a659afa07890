"""ctypes loader of libdswarm_cuda.so.

The library is built in-tree by ``ops/_build.py`` (nvcc, sm_100a).  On a box
with a GPU a missing or unloadable library is an error: there is no silent
fallback to library ops on the paths that name these kernels.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _build

_cuda = None

c_void_p, c_int, c_ll, c_float, c_uint = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_uint
c_size_t = ctypes.c_size_t

_SIGS = {
    "dsw_gemm_bf16": [c_void_p, c_ll, c_int, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_ll,
                      c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p],
    "dsw_layernorm_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "dsw_layernorm_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_int, c_int, c_void_p],
    "dsw_layernorm_bwd_blocks": [c_int],
    "dsw_colsum_accum": [c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p],
    "dsw_embedding_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "dsw_embedding_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "dsw_embedding_bwd_sorted": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "dsw_mask_count": [c_void_p, c_int, c_void_p, c_void_p],
    "dsw_cross_entropy": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int,
                          c_void_p, c_void_p],
    "dsw_cast_f32_bf16": [c_void_p, c_void_p, c_ll, c_void_p],
    "dsw_cast_bf16_f32": [c_void_p, c_void_p, c_ll, c_void_p],
    "dsw_sumsq": [c_void_p, c_ll, c_void_p, c_void_p],
    "dsw_clip_coef": [c_void_p, c_float, c_void_p],
    "dsw_adamw": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_float, c_float, c_float,
                  c_int, c_void_p, c_int, c_void_p],
    "dsw_sgd": [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_int, c_void_p, c_int, c_void_p],
    "dsw_symm_alloc": [c_size_t, ctypes.POINTER(c_void_p)],
    "dsw_symm_free": [c_void_p],
    "dsw_symm_export": [c_void_p, c_void_p],
    "dsw_symm_import": [c_void_p, ctypes.POINTER(c_void_p)],
    "dsw_symm_unimport": [c_void_p],
    "dsw_max_peers": [],
    "dsw_stream_wait_geq32": [c_void_p, c_uint, c_void_p],
    "dsw_stream_write32": [c_void_p, c_uint, c_void_p],
    "dsw_copy_async": [c_void_p, c_void_p, c_size_t, c_void_p],
    "dsw_outer_sync": [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_float, c_float, c_int,
                       c_uint, c_ll, c_int, c_int, c_void_p, c_void_p],
    "dsw_grad_allreduce": [c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_ll, c_int, c_int, c_int, c_uint, c_ll, c_int,
                           c_int, c_int, c_void_p, c_void_p],
    "dsw_outer_sync_nvls": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_float,
                            c_float, c_int, c_uint, c_ll, c_int, c_void_p, c_void_p],
    "dsw_grad_allreduce_nvls": [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_ll, c_int, c_int, c_int, c_uint,
                                c_ll, c_int, c_void_p, c_void_p],
    "dsw_attention_fwd": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "dsw_attention_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_int, c_float, c_void_p, c_void_p],
}


def cuda_lib():
    """The loaded kernel library.  It is rebuilt first when a source or header under csrc/ is newer than
    it (a cheap time-stamp check; the build itself is serialised between processes by a file lock).
    ``DSWARM_LIB_VARIANT=trace|bounds`` selects one of the debugging builds (ops/_build.py)."""
    global _cuda
    if _cuda is None:
        variant = os.environ.get("DSWARM_LIB_VARIANT", "")
        path = _build.build_cuda(force=os.environ.get("DSWARM_REBUILD", "0") == "1", variant=variant)
        lib = ctypes.CDLL(path)
        for name, argtypes in _SIGS.items():
            fn = getattr(lib, name, None)
            if fn is None:
                continue
            fn.restype = c_int
            fn.argtypes = argtypes
        _cuda = lib
    return _cuda


_loaded = False


def load_all_kernels() -> None:
    """Load every kernel of the library on the current device now.  A kernel's
    first launch may otherwise wait for the device to go idle, which deadlocks
    when a pipeline receive is already spinning there (see the package __init__)."""
    global _loaded
    if _loaded:
        return
    lib = cuda_lib()
    for name in ("dsw_load_gemm", "dsw_load_elementwise", "dsw_load_optim", "dsw_load_collectives",
                 "dsw_load_attention"):
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.restype = c_int
            fn.argtypes = []
            if fn() != 0:
                raise RuntimeError(f"{name} failed")
    _loaded = True


def stream_ptr(stream: Optional[torch.cuda.Stream] = None) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


LAUNCHES = 0   # launcher calls so far (each launches at least one kernel of this library)


def check(rc: int, what: str) -> None:
    global LAUNCHES
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
    LAUNCHES += 1


def launch_count() -> int:
    return LAUNCHES


_STATUS_TEXT = {1: "an mbarrier wait ran out inside a kernel",
                2: "a wait for a peer GPU ran out inside a fused collective",
                3: "a kernel saw an out-of-range index (token id or target)"}


class Status:
    """Device status word shared by the kernels of one engine.  Kernels that
    give up on a wait write a code here instead of hanging; ``raise_if_set``
    turns it into an exception at a point where the host synchronises anyway."""

    def __init__(self, device: torch.device):
        self.word = torch.zeros(1, dtype=torch.int32, device=device)

    @property
    def ptr(self) -> int:
        return self.word.data_ptr()

    def read(self) -> int:
        return int(self.word.item())

    def raise_if_set(self) -> None:
        code = self.read()
        if code != 0:
            self.word.zero_()
            raise RuntimeError(f"kernel status {code}: {_STATUS_TEXT.get(code, 'unknown')}")
