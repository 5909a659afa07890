"""Symmetric (peer-mapped) device buffers for a stage's replicas.

Every replica allocates a buffer of the same size with cudaMalloc, exports a
CUDA IPC handle, and opens the handles of the other replicas of its stage
(all on one NVSwitch node), which yields R device pointers to the same logical
buffer.  The fused collectives (csrc/collectives.cu) take these pointers and
issue plain peer loads and stores.  The reference has no counterpart: it
copies through host memory and gloo (src/comm.py:38,117-123).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops._lib import check, cuda_lib

MAX_PEERS = 8
FLAG_BLOCKS = 148          # csrc/dswarm.h: DSW_MAX_COLL_BLOCKS
FLAG_WORDS = FLAG_BLOCKS * MAX_PEERS
GUARD_BYTES = 256          # canary zone in front of and behind every symmetric buffer
CANARY = 0xC5


class CanaryError(RuntimeError):
    """Something wrote outside a symmetric buffer (into the guard zone in front of or behind it)."""


class _CudaArray:
    """Minimal __cuda_array_interface__ carrier so torch can view raw device memory."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
        self._owner = owner


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``group`` plus pointers to
    the peers' copies.  ``local`` is this rank's buffer as a uint8 tensor."""

    def __init__(self, nbytes: int, device: torch.device, group=None, ranks: Optional[Sequence[int]] = None,
                 multicast: bool = False):
        """``multicast``: also bind the replicas' buffers to an NVLink multicast object, so that kernels can
        reduce and broadcast inside the NVSwitch through ``mc_ptr`` (``multimem`` instructions).  Such memory
        comes from the driver's virtual-memory API; PyTorch's symmetric-memory allocator is used for that
        plumbing (allocation, handle exchange, binding), the kernels on it are this library's.  ``mc_ptr`` is 0
        when the replicas cannot form a multicast group (one replica, or no NVLS on the box)."""
        lib = cuda_lib()
        self.device = device
        self.nbytes = (nbytes + 255) // 256 * 256
        self.mc_ptr = 0
        self._symm_handle = None
        if multicast and group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
            self._init_multicast(device, group)
            return
        # Peers store into these buffers with plain pointers, and the sanitizer tools are closed on shared GPUs,
        # so every buffer sits between two guard zones filled with a fixed byte; check_canaries() (called when
        # the buffer is closed, and per step with DSWARM_CANARY_CHECK=1) tells whether a store went astray.
        p = ctypes.c_void_p()
        with torch.cuda.device(device):
            check(lib.dsw_symm_alloc(self.nbytes + 2 * GUARD_BYTES, ctypes.byref(p)), "dsw_symm_alloc")
        self._base = p.value
        self.ptr = self._base + GUARD_BYTES
        self._imported: List[int] = []
        self._whole = torch.as_tensor(_CudaArray(self._base, self.nbytes + 2 * GUARD_BYTES, self), device=device)
        self._whole[:GUARD_BYTES].fill_(CANARY)
        self._whole[GUARD_BYTES + self.nbytes:].fill_(CANARY)
        self.local = self._whole[GUARD_BYTES:GUARD_BYTES + self.nbytes]
        R = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank_in_group = dist.get_rank(group) if R > 1 else 0
        self.peer_ptrs: List[int] = [self.ptr]
        if R > 1:
            if R > MAX_PEERS:
                raise ValueError(f"at most {MAX_PEERS} replicas per stage")
            handle = (ctypes.c_char * 64)()
            check(lib.dsw_symm_export(self._base, handle), "dsw_symm_export")
            mine = torch.frombuffer(bytearray(handle.raw), dtype=torch.uint8).to(device)
            gathered = [torch.empty_like(mine) for _ in range(R)]
            dist.all_gather(gathered, mine, group=group)
            self.peer_ptrs = []
            for j, h in enumerate(gathered):
                if j == self.rank_in_group:
                    self.peer_ptrs.append(self.ptr)
                    continue
                raw = bytes(h.cpu().numpy().tobytes())
                q = ctypes.c_void_p()
                with torch.cuda.device(device):
                    check(lib.dsw_symm_import(raw, ctypes.byref(q)), "dsw_symm_import")
                self._imported.append(q.value)
                self.peer_ptrs.append(q.value + GUARD_BYTES)        # the peer's payload starts behind its front guard
        self.R = R
        self._table = (ctypes.c_void_p * MAX_PEERS)(*[ctypes.c_void_p(x) for x in self.peer_ptrs])

    def _init_multicast(self, device: torch.device, group) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        total = self.nbytes + 2 * GUARD_BYTES
        with torch.cuda.device(device):
            whole = symm_mem.empty(total, dtype=torch.uint8, device=device)
            whole.zero_()
            hdl = symm_mem.rendezvous(whole, group)
        self._symm_handle = hdl
        self._whole = whole
        self._base = whole.data_ptr()
        self.ptr = self._base + GUARD_BYTES
        self._imported = []
        self._whole[:GUARD_BYTES].fill_(CANARY)
        self._whole[GUARD_BYTES + self.nbytes:].fill_(CANARY)
        self.local = self._whole[GUARD_BYTES:GUARD_BYTES + self.nbytes]
        self.R = dist.get_world_size(group)
        self.rank_in_group = dist.get_rank(group)
        if self.R > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS} replicas per stage")
        self.peer_ptrs = [int(p) + GUARD_BYTES for p in hdl.buffer_ptrs]
        assert self.peer_ptrs[self.rank_in_group] == self.ptr
        mc = int(hdl.multicast_ptr or 0)                   # 0 where the replicas cannot form a multicast group
        self.mc_ptr = mc + GUARD_BYTES if mc else 0
        self._table = (ctypes.c_void_p * MAX_PEERS)(*[ctypes.c_void_p(x) for x in self.peer_ptrs])
        torch.cuda.synchronize(device)
        dist.barrier(group=group, device_ids=[device.index])      # every replica's guards and zeros are in place

    @property
    def table(self):
        """Host array of R device pointers in replica order (launcher argument)."""
        return self._table

    def view(self, dtype: torch.dtype, numel: Optional[int] = None, byte_offset: int = 0) -> torch.Tensor:
        t = self.local[byte_offset:].view(dtype)
        return t if numel is None else t[:numel]

    def check_canaries(self) -> None:
        """Raise ``CanaryError`` if a guard zone of this rank's buffer no longer holds the canary byte
        (one small device-to-host read; synchronises the current stream)."""
        if not self._base:
            return
        front = self._whole[:GUARD_BYTES]
        back = self._whole[GUARD_BYTES + self.nbytes:]
        bad = [name for name, z in (("in front of", front), ("behind", back)) if not bool((z == CANARY).all())]
        if bad:
            raise CanaryError(f"the guard zone {' and '.join(bad)} a symmetric buffer of {self.nbytes} bytes was "
                              "overwritten: a kernel stored outside the buffer")

    def close(self) -> None:
        lib = cuda_lib()
        for q in self._imported:
            lib.dsw_symm_unimport(q)
        self._imported = []
        if self._base:
            try:
                self.check_canaries()
            finally:
                self.local = self._whole = None
                if self._symm_handle is None:
                    lib.dsw_symm_free(self._base)
                self._symm_handle = None              # multicast-bound memory goes back with its tensor
                self._base = self.ptr = 0


class LocalPeerSet:
    """R buffers on ONE GPU standing in for R replicas.  Used to check the
    collective kernels' arithmetic with sequential launches (one per emulated
    replica, barriers off): kernels that wait on one another must not share a GPU."""

    def __init__(self, tensors: Sequence[torch.Tensor]):
        self.tensors = list(tensors)
        self.R = len(tensors)
        self._table = (ctypes.c_void_p * MAX_PEERS)(*[ctypes.c_void_p(t.data_ptr()) for t in tensors])

    @property
    def table(self):
        return self._table
