"""Encoder interface of the distributed multimodal encoder service and its wire format.

``BaseEncoder`` mirrors the reference ABC (teletron/core/distributed/base_encoder.py:18-82):
``setup()`` loads models, ``encode(raw_batch) -> (tensors, size_info)``, ``get_output_schema()``
names the tensors, ``_pack_tensors`` flattens them into one bf16 blob.

Wire format (one message pair per sample, NCCL/gloo p2p):
  header  int32[HEADER_INTS] = [MAGIC, VERSION, seq_no, n_tensors, flags, then per tensor (ndim, d0..d4)]
  payload flat bf16 = the tensors flattened in schema order
After an early stop request the producer closes each stream with one header that carries ``FLAG_STOP`` and no payload,
which completes the header receive the consumer keeps in flight.  ``FLAG_NEXT_SAME`` on a header promises that the
next message is a full sample of the same shapes: the consumer then posts both of its receives (into a second
buffer) while the current sample trains, which is what makes the hand-off double-buffered.
A fixed, versioned header replaces the reference's bare int32[16] of concatenated shapes
(teletron/train/consumer_dataloader.py:106-122), whose length silently disagreed between
producer and consumer once a fifth tensor (shared noise) was added.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Dict, List, Sequence, Tuple

import torch

MAGIC = 0x7E1E7204 & 0x7FFFFFFF
VERSION = 2
HEADER_INTS = 64
MAX_TENSORS = 9
MAX_DIMS = 5
FLAG_LAST = 1
FLAG_STOP = 2   # header without a payload: the producer was asked to stop and will send nothing more
FLAG_NEXT_SAME = 4  # a promise: another full sample with the same shapes follows, whatever happens (also after a stop
                    # request), so the consumer may post the receives of its header AND payload right away


def encode_header(shapes: Sequence[Sequence[int]], seq_no: int, flags: int = 0) -> torch.Tensor:
    if len(shapes) > MAX_TENSORS:
        raise ValueError(f"at most {MAX_TENSORS} tensors per message, got {len(shapes)}")
    h = torch.zeros(HEADER_INTS, dtype=torch.int32)
    h[0], h[1], h[2], h[3], h[4] = MAGIC, VERSION, seq_no & 0x7FFFFFFF, len(shapes), flags
    pos = 5
    for s in shapes:
        if len(s) > MAX_DIMS:
            raise ValueError(f"tensor rank {len(s)} exceeds {MAX_DIMS}")
        h[pos] = len(s)
        for i, d in enumerate(s):
            h[pos + 1 + i] = int(d)
        pos += 1 + MAX_DIMS
    return h


def decode_header(h: torch.Tensor) -> Tuple[List[Tuple[int, ...]], int, int]:
    """Returns (shapes, seq_no, flags); raises ValueError on a corrupt or foreign header."""
    v = h.tolist()
    if len(v) != HEADER_INTS or v[0] != MAGIC:
        raise ValueError("encoder message header has a bad magic number (corrupt or out-of-sync stream)")
    if v[1] != VERSION:
        raise ValueError(f"encoder message header version {v[1]} != {VERSION}")
    n = v[3]
    if not 0 <= n <= MAX_TENSORS:
        raise ValueError(f"encoder message header names {n} tensors")
    shapes, pos = [], 5
    for _ in range(n):
        nd = v[pos]
        if not 0 <= nd <= MAX_DIMS:
            raise ValueError("encoder message header has an invalid rank field")
        dims = tuple(int(d) for d in v[pos + 1: pos + 1 + nd])
        if any(d < 0 for d in dims):
            raise ValueError("encoder message header has a negative extent")
        shapes.append(dims)
        pos += 1 + MAX_DIMS
    return shapes, v[2], v[4]


def numel_of(shapes) -> int:
    total = 0
    for s in shapes:
        n = 1
        for d in s:
            n *= d
        total += n
    return total


def pack_tensors(tensors: Sequence[torch.Tensor], dtype=torch.bfloat16) -> torch.Tensor:
    return torch.cat([t.reshape(-1).to(dtype) for t in tensors])


def unpack_tensors(blob: torch.Tensor, shapes) -> List[torch.Tensor]:
    want = numel_of(shapes)
    if want != blob.numel():
        raise ValueError(f"payload has {blob.numel()} elements but the header describes {want}")
    out, pos = [], 0
    for s in shapes:
        n = 1
        for d in s:
            n *= d
        out.append(blob[pos:pos + n].view(*s))
        pos += n
    return out


class BaseEncoder(ABC):
    """One encoder rank's model bundle. Subclasses register with ``ENCODERS.register(name)``."""

    def __init__(self, device=None, **kwargs):
        self.device = device
        self.kwargs = kwargs

    @abstractmethod
    def setup(self) -> None:
        """Load / build the encoder models on ``self.device``."""

    @abstractmethod
    def encode(self, raw_batch) -> Tuple[List[torch.Tensor], torch.Tensor]:
        """raw dataset batch -> (tensors in schema order, header tensor)."""

    @abstractmethod
    def get_output_schema(self) -> List[str]:
        """Names of the tensors ``encode`` returns, in order."""

    def _pack_tensors(self, tensors):
        return pack_tensors(tensors)

    def _get_tensors_size(self, tensors, seq_no: int = 0, flags: int = 0):
        return encode_header([tuple(t.shape) for t in tensors], seq_no, flags)

    def as_dict(self, tensors) -> Dict[str, torch.Tensor]:
        return dict(zip(self.get_output_schema(), tensors))
