"""The copy-engine pipeline transport (parallel/ce_comm.py) on the CPU: its own Python code runs unchanged for
every rank of a swarm inside one process, against an emulation of the three stream operations it issues
(wait until a 32-bit word reaches a value, write a word, copy bytes).  The emulated device then executes the
queued operations of all streams in a random interleaving.  Checked: every receive ends up with the payload of
the matching send (inbox slot addressing, peer indices, flag words), rings of four slots carry far more than
four messages per pair without overwriting an unread one, and nothing deadlocks."""
import ctypes
import random
import types

import pytest
import torch

import diloco_swarm_b200.parallel.ce_comm as ce


class _Device:
    """Streams of all ranks: a queue of operations each; `run` executes them in a random order that respects
    every stream's own order and the waits."""

    def __init__(self, rng):
        self.rng = rng
        self.queues = {}
        self.done = {}
        self.current = {}              # rank -> its compute stream
        self.rank = 0
        self.next_id = 1

    def new_stream(self):
        sid = self.next_id
        self.next_id += 1
        self.queues[sid], self.done[sid] = [], 0
        return sid

    def run(self):
        while any(self.done[s] < len(q) for s, q in self.queues.items()):
            ready = []
            for s, q in self.queues.items():
                if self.done[s] == len(q):
                    continue
                op = q[self.done[s]]
                if op[0] == "wait" and ctypes.c_uint32.from_address(op[1]).value < op[2]:
                    continue
                if op[0] == "after" and self.done[op[1]] < op[2]:
                    continue
                ready.append(s)
            assert ready, "the queued stream operations deadlock"
            s = self.rng.choice(ready)
            op = self.queues[s][self.done[s]]
            if op[0] == "write":
                ctypes.c_uint32.from_address(op[1]).value = op[2]
            elif op[0] == "copy":
                ctypes.memmove(op[1], op[2], op[3])
            self.done[s] += 1


class _Stream:
    dev = None

    def __init__(self, device=None):
        self.cuda_stream = _Stream.dev.new_stream()

    def wait_stream(self, other):
        d = _Stream.dev
        d.queues[self.cuda_stream].append(("after", other.cuda_stream, len(d.queues[other.cuda_stream])))


class _Lib:
    def __init__(self, dev):
        self.dev = dev

    def dsw_stream_wait_geq32(self, addr, value, st):
        self.dev.queues[st].append(("wait", addr, value))
        return 0

    def dsw_stream_write32(self, addr, value, st):
        self.dev.queues[st].append(("write", addr, value))
        return 0

    def dsw_copy_async(self, dst, src, n, st):
        self.dev.queues[st].append(("copy", dst, src, n))
        return 0


class _Box:
    registry = {}

    def __init__(self, nbytes, device, group):
        self.mem = torch.zeros(nbytes, dtype=torch.uint8)
        self.ptr = self.mem.data_ptr()
        self.rank = _Stream.dev.rank
        _Box.registry[self.rank] = self

    @property
    def peer_ptrs(self):
        return {r: b.ptr for r, b in _Box.registry.items()}

    def close(self):
        pass


def _world(rank, S, R):
    stage2ranks = {s: [r for r in range(S * R) if r % S == s] for s in range(S)}
    return types.SimpleNamespace(rank=rank, world_size=S * R, num_stages=S, stage=rank % S, stage2ranks=stage2ranks)


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("S,R", [(2, 1), (2, 2), (2, 4), (4, 2), (3, 2)])
def test_every_message_arrives_in_its_slot(S, R, seed, monkeypatch):
    rng = random.Random(100 * S + 10 * R + seed)
    dev = _Device(rng)
    _Stream.dev = dev
    _Box.registry = {}
    monkeypatch.setattr(ce, "SymmetricBuffer", _Box)
    monkeypatch.setattr(ce, "cuda_lib", lambda: _Lib(dev))
    monkeypatch.setattr(ce, "stream_ptr", lambda: dev.current[dev.rank].cuda_stream)
    monkeypatch.setattr(torch.cuda, "Stream", _Stream)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda *a, **k: dev.current[dev.rank])
    monkeypatch.setattr(torch.Tensor, "record_stream", lambda self, s: None, raising=False)
    monkeypatch.setattr(ce.dist, "group", types.SimpleNamespace(WORLD=None), raising=False)
    n = S * R
    shape = (3, 5, 8)                                       # 120 bf16 = 240 bytes: padded to a 256-byte slot
    comms = []
    for r in range(n):
        dev.rank = r
        dev.current[r] = _Stream()
        comms.append(ce.CopyEngineComm(_world(r, S, R), shape, torch.bfloat16, torch.device("cpu"), slots=4))
    # a causal global order of messages between ranks of adjacent stages, both directions, up to 14 per pair
    pairs = [(a, b) for a in range(n) for b in range(n) if abs(a % S - b % S) == 1]
    msgs = [p for p in pairs for _ in range(rng.randint(0, 14))]
    rng.shuffle(msgs)
    sent, got, keep = {}, [], []
    for i, (src, dst) in enumerate(msgs):
        payload = torch.full(shape, float(i % 250), dtype=torch.bfloat16)
        keep.append(payload)
        dev.rank = src
        comms[src].send_forward(payload, dst) if dst % S > src % S else comms[src].send_backward(payload, dst)
        sent.setdefault((src, dst), []).append(i)
        dev.rank = dst
        comms[dst]._src = {0: src}
        got.append((i, comms[dst].recv(0)))
    dev.run()
    for i, out in got:
        assert torch.all(out.float() == float(i % 250)), f"message {i} {msgs[i]} arrived as {out.flatten()[0].item()}"
    for c in comms:                                         # counters agree on both ends of every pair
        for q, k in c.sent.items():
            assert comms[q].got[c.world.rank] == k
