"""Symmetric peer memory for kernel-initiated communication inside one NVLink/NVSwitch box.

``SymmetricArena`` allocates buffers with ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations whose handles are exchanged through the process group's store), so every rank holds
a device pointer to every peer's copy.  Kernels receive those pointers and move data with plain
loads and stores over NVLink; ordering between ranks uses the epoch-numbered flag barrier of
``csrc/comm.cu`` (bounded spin, status word on time-out).  The reference has no counterpart: it
only calls NCCL collectives (teletron/core/parallel_state.py:384-633).

Only ordinary per-thread loads and stores (and non-broadcast TMA) ever touch these buffers.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib

_SLOTS = 8


def symmetric_memory_available() -> bool:
    if not torch.cuda.is_available() or not dist.is_initialized():
        return False
    try:
        import importlib

        importlib.import_module("torch.distributed._symmetric_memory")
        return True
    except Exception:
        return False


class SymmTensor:
    """A local tensor plus the device addresses of the same buffer on every rank of the group."""

    def __init__(self, tensor: torch.Tensor, peer_ptrs: List[int], handle):
        self.tensor = tensor
        self.peer_ptrs = list(peer_ptrs)
        self.handle = handle
        self._c = (_lib.c_ll * len(self.peer_ptrs))(*self.peer_ptrs)

    def c_ptrs(self, elem_offset: int = 0):
        """ctypes array of peer addresses, optionally advanced by ``elem_offset`` elements."""
        if elem_offset == 0:
            return self._c
        b = elem_offset * self.tensor.element_size()
        return (_lib.c_ll * len(self.peer_ptrs))(*[p + b for p in self.peer_ptrs])


class SymmetricArena:
    def __init__(self, group=None, timeout_ms: int = 20000):
        import torch.distributed._symmetric_memory as symm_mem

        self._sm = symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.timeout_ms = timeout_ms
        self.device = torch.device("cuda", torch.cuda.current_device())
        L = _lib.lib()
        self.max_peers = L.tt_comm_max_peers()
        if self.world > self.max_peers:
            raise RuntimeError(f"symmetric arena supports at most {self.max_peers} ranks, got {self.world}")
        try:
            symm_mem.enable_symm_mem_for_group(self.group.group_name)
        except Exception:
            pass
        self.flags = self.alloc(self.max_peers * _SLOTS, torch.int32)
        self.flags.tensor.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)  # everybody's flags are zero before the first device barrier
        self._epoch = [0] * _SLOTS

    def alloc(self, numel: int, dtype: torch.dtype) -> SymmTensor:
        t = self._sm.empty(int(numel), dtype=dtype, device=self.device)
        h = self._sm.rendezvous(t, self.group)
        return SymmTensor(t, [int(p) for p in h.buffer_ptrs], h)

    def barrier(self, slot: int = 0):
        """Device-side barrier on the current stream across the group's GPUs."""
        self._epoch[slot] = (self._epoch[slot] + 1) & 0x7FFFFFFF
        rc = _lib.lib().tt_peer_barrier(self.flags.c_ptrs(), _lib.c_int(self.world), _lib.c_int(self.rank),
                                        _lib.c_int(slot), _lib.c_uint(self._epoch[slot]),
                                        _lib.c_int(self.timeout_ms), _lib.ptr(_lib.status_word(self.device)),
                                        _lib.stream())
        _lib.check(rc, "tt_peer_barrier")
