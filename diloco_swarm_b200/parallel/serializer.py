"""Message framing for transports that do not know their sender in advance.

The reference prepends a whole extra plane of the tensor's shape to carry two
numbers, (root_rank, local_micro_step), which doubles every pipeline message
(src/serializer.py:9-15).  The default pipeline engine of this package needs no
framing at all: routing is a pure function of (seed, step), so both ends know
which microbatch a transfer belongs to (parallel/schedule.py).  This class is
the compact equivalent for transports that still want self-describing
messages (receive-from-any experiments, logging of traffic): a 16-byte header
in front of the flat payload instead of a second plane.
"""
from __future__ import annotations

from typing import Tuple

import torch

Metadata = Tuple[int, int]          # (root_rank, local_micro_step)
HEADER_BYTES = 16


class Serializer:
    def __init__(self, shape: Tuple[int, ...], dtype: torch.dtype = torch.float32):
        self.payload_shape, self.dtype = tuple(shape), dtype
        n = 1
        for s in shape:
            n *= s
        self.payload_bytes = n * torch.empty((), dtype=dtype).element_size()
        self.shape = (HEADER_BYTES + self.payload_bytes,)      # uint8 message

    def serialize(self, tensor: torch.Tensor, metadata: Metadata) -> torch.Tensor:
        assert tuple(tensor.shape) == self.payload_shape and tensor.dtype == self.dtype
        msg = torch.empty(self.shape, dtype=torch.uint8, device=tensor.device)
        head = torch.tensor([metadata[0], metadata[1]], dtype=torch.int64)
        msg[:HEADER_BYTES] = head.view(torch.uint8).to(tensor.device)
        msg[HEADER_BYTES:] = tensor.detach().contiguous().view(-1).view(torch.uint8)
        return msg

    def deserialize(self, msg: torch.Tensor) -> Tuple[torch.Tensor, Metadata]:
        head = msg[:HEADER_BYTES].cpu().view(torch.int64)
        payload = msg[HEADER_BYTES:].view(self.dtype).view(self.payload_shape)
        return payload, (int(head[0]), int(head[1]))
