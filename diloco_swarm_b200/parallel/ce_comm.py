"""Pipeline point-to-point transport on the copy engines, with stream-ordered flags.

The reference moves activations through host memory and gloo (src/comm.py:16-115).
The NCCL transport of ``parallel/comm.py`` keeps them on the device, but every NCCL
send or receive is a kernel that spins on the GPU until its partner shows up, and a
persistent GEMM whose tiles are assigned statically needs every SM: one SM held by a
waiting transfer turns the GEMM into two waves.  Measured on a 2 x 1 pipeline, the
stage that had such kernels resident ran its microbatches 20 % slower (9.8 instead
of 8.1 ms), and the forwards of the fill phase 65 % slower.

Here no kernel is involved in a transfer at all:

* every rank owns an *inbox* in a peer-mapped buffer: per possible sender a ring of
  ``slots`` message slots, plus two small flag arrays;
* the sender copies the tensor into its ring in the receiver's inbox with a
  device-to-device ``cudaMemcpyAsync`` on a copy stream (NVLink, copy engines) and
  then writes the message number into the receiver's ``arrived`` flag with a stream
  memory operation; before reusing a slot its stream waits, again with a stream
  memory operation, until the receiver's ``consumed`` count says the slot is free;
* the receiver's compute stream waits for the ``arrived`` flag, copies the slot into
  a tensor of its own and writes ``consumed`` back into the sender's memory.

Messages of one (sender, receiver) pair are consumed in the order they were sent,
which is the order the static plans guarantee (``schedule.check_plans``).  Nothing
has to be posted ahead of time: a message lands whether or not the receiver has
got to it yet, so the sender only ever waits when a ring is full.  A wait is a
stream wait, not a spinning kernel; it ends when the peer writes the flag (or with
the process).  One node only: the inboxes are CUDA-IPC mappings.
"""
from __future__ import annotations

import math
import os
import time
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops._lib import cuda_lib, stream_ptr
from .schedule import BWD, FWD, FWD_BWD, Op
from .symm import MAX_PEERS, SymmetricBuffer

FLAG_BYTES = 4096            # arrived[] at +0, consumed[] at +2048 (one uint32 per adjacent-stage peer)


def check(rc: int, what: str) -> None:
    """These calls queue copies and stream memory operations, not kernels: they stay out of the launch count."""
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


class CopyEngineComm:
    device_async = True       # the host queues transfers; completion is a matter of the device streams

    def __init__(self, world, shape: Tuple[int, ...], dtype: torch.dtype, device: torch.device, slots: int = 4):
        self.world, self.shape, self.dtype, self.device = world, tuple(shape), dtype, device
        self.slots = max(1, slots)
        self.tolerant = False
        self.bytes_sent = 0
        self.deadline: Optional[float] = None
        self.prefetch = 0
        w = world
        self.active = w.num_stages > 1
        if not self.active:
            return
        if w.world_size > MAX_PEERS:
            raise ValueError(f"the copy-engine transport maps every rank's inbox: at most {MAX_PEERS} ranks on one node")
        self.nbytes = math.prod(self.shape) * torch.empty((), dtype=dtype).element_size()
        self.msg_bytes = (self.nbytes + 255) // 256 * 256
        # adjacent-stage peers in one fixed order, the same on both ends of a pair
        self.peers: List[int] = []
        if w.stage > 0:
            self.peers += list(w.stage2ranks[w.stage - 1])
        if w.stage + 1 < w.num_stages:
            self.peers += list(w.stage2ranks[w.stage + 1])
        self.index = {q: i for i, q in enumerate(self.peers)}
        self.region = self.slots * self.msg_bytes
        # every rank's inbox has the same size (the largest any rank needs), so one all-gather of handles maps all
        S = w.num_stages
        most = max((len(w.stage2ranks[s - 1]) if s > 0 else 0) + (len(w.stage2ranks[s + 1]) if s + 1 < S else 0)
                   for s in range(S))
        self.flag_off = most * self.region
        self.box = SymmetricBuffer(self.flag_off + FLAG_BYTES, device, dist.group.WORLD)
        self.sent: Dict[int, int] = {q: 0 for q in self.peers}        # messages sent to q so far
        self.got: Dict[int, int] = {q: 0 for q in self.peers}         # messages consumed from q so far
        self.copy_streams: Dict[int, torch.cuda.Stream] = {q: torch.cuda.Stream(device) for q in self.peers}
        self._lib = cuda_lib()
        # A flag in a peer's memory is written either directly by a stream memory operation on the mapped address
        # or, the default, by writing a local staging word and copying its four bytes over (same stream, so in
        # order): the second form uses nothing but a plain peer copy.
        self.direct_flags = os.environ.get("DSWARM_CE_DIRECT_FLAGS", "0") == "1"
        self._stage = torch.zeros(2 * len(self.peers) + 2, dtype=torch.int32, device=device)

    def _remote_write(self, addr: int, value: int, stage_word: int, st: int) -> None:
        lib = self._lib
        if self.direct_flags:
            check(lib.dsw_stream_write32(addr, value, st), "dsw_stream_write32")
            return
        local = self._stage.data_ptr() + 4 * stage_word
        check(lib.dsw_stream_write32(local, value, st), "dsw_stream_write32")
        check(lib.dsw_copy_async(addr, local, 4, st), "dsw_copy_async")

    # -- addresses ---------------------------------------------------------------
    def _peer_index_of_me(self, q: int) -> int:
        """Where this rank sits in rank q's list of adjacent-stage peers (q computes the same list)."""
        w = self.world
        sq = q % w.num_stages
        lst: List[int] = []
        if sq > 0:
            lst += list(w.stage2ranks[sq - 1])
        if sq + 1 < w.num_stages:
            lst += list(w.stage2ranks[sq + 1])
        return lst.index(w.rank)

    def _slot_in(self, base: int, sender_index: int, k: int) -> int:
        return base + sender_index * self.region + (k % self.slots) * self.msg_bytes

    # -- PipelineComm interface ------------------------------------------------------
    def warmup(self) -> None:
        """Nothing is created lazily here; one barrier makes sure every inbox is mapped before the first send."""
        if self.active:
            dist.barrier(device_ids=[self.device.index])

    def begin_step(self, ops: Sequence[Op], timeout_s: Optional[float] = None) -> None:
        w = self.world
        self._src: Dict[int, int] = {}
        for i, op in enumerate(ops):
            if op.kind in (FWD, FWD_BWD) and op.prev >= 0:
                self._src[i] = op.prev
            elif op.kind == BWD and op.next >= 0:
                self._src[i] = op.next
        self.deadline = time.time() + timeout_s if timeout_s else None

    def tick(self, op_index: int) -> None:
        """Nothing to post: messages land in the inbox whether or not the receiver has got to them."""

    def recv(self, op_index: int) -> torch.Tensor:
        src = self._src[op_index]
        k = self.got[src]
        self.got[src] = k + 1
        i = self.index[src]
        st = stream_ptr()
        lib, base = self._lib, self.box.ptr
        check(lib.dsw_stream_wait_geq32(base + self.flag_off + 4 * i, k + 1, st), "dsw_stream_wait_geq32")
        out = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        check(lib.dsw_copy_async(out.data_ptr(), self._slot_in(base, i, k), self.nbytes, st), "dsw_copy_async")
        # tell the sender that this slot is free again (its memory, our stream: after the copy)
        peer = self.box.peer_ptrs[src]
        self._remote_write(peer + self.flag_off + 2048 + 4 * self._peer_index_of_me(src), k + 1, len(self.peers) + i, st)
        return out

    def send_forward(self, tensor: torch.Tensor, dst: int) -> None:
        self._send(tensor, dst)

    def send_backward(self, tensor: torch.Tensor, dst: int) -> None:
        self._send(tensor, dst)

    def _send(self, tensor: torch.Tensor, dst: int) -> None:
        t = tensor.detach()
        if t.dtype != self.dtype:
            t = t.to(self.dtype)
        t = t.contiguous()
        assert t.numel() * t.element_size() == self.nbytes, "pipeline messages have one fixed shape"
        k = self.sent[dst]
        self.sent[dst] = k + 1
        cs = self.copy_streams[dst]
        cs.wait_stream(torch.cuda.current_stream())          # the tensor has been produced
        t.record_stream(cs)                                  # its memory is not reused before the copy has run
        st = cs.cuda_stream
        lib = self._lib
        if k >= self.slots:                                   # the slot's previous message has been consumed
            check(lib.dsw_stream_wait_geq32(self.box.ptr + self.flag_off + 2048 + 4 * self.index[dst],
                                            k - self.slots + 1, st), "dsw_stream_wait_geq32")
        peer = self.box.peer_ptrs[dst]
        me = self._peer_index_of_me(dst)
        check(lib.dsw_copy_async(self._slot_in(peer, me, k), t.data_ptr(), self.nbytes, st), "dsw_copy_async")
        self._remote_write(peer + self.flag_off + 4 * me, k + 1, self.index[dst], st)
        self.bytes_sent += self.nbytes

    def end_step(self) -> None:
        """Sends drain on their own streams; nothing on the compute stream depends on them."""

    def abandon_step(self) -> None:
        pass

    def close(self) -> None:
        if self.active:
            torch.cuda.synchronize(self.device)
            self.box.close()
            self.active = False
