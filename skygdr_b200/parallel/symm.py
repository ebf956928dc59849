"""Symmetric heap over CUDA IPC: every rank allocates the same region and maps every peer's.

This is the set-up handshake of a flow between GPUs: what the reference does per connection with
``ConnInfo`` / rkey / address exchanges over TCP before RDMA can start (src/cpu_client.cc:618-665,
src/gpu_server.cu:293-323) happens here once per process group, with CUDA IPC handles exchanged over
``torch.distributed``; after that kernels store into peers' memory through plain pointers.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from .._ext import load


class SymmetricHeap:
    def __init__(self, nbytes: int, rank: int, world: int, device: torch.device, group=None):
        self._C = load()
        self.rank, self.world, self.device, self.nbytes = rank, world, device, nbytes
        self.local_ptr, handle = self._C.ipc_alloc(nbytes)
        if world > 1:
            handles: List[bytes] = [b""] * world
            dist.all_gather_object(handles, bytes(handle), group=group)
            self.ptrs = [self.local_ptr if r == rank else self._C.ipc_open(handles[r]) for r in range(world)]
        else:
            self.ptrs = [self.local_ptr]
        self._offsets: Dict[str, Tuple[int, int]] = {}
        self._top = 0

    def alloc(self, name: str, nbytes: int, align: int = 256, local: bool = True) -> int:
        """Reserves a named range; every rank must make the same calls in the same order. ``local=False`` records a
        range that exists only on peers with a larger heap (ranks with different roles may size their heaps differently)."""
        off = (self._top + align - 1) // align * align
        assert not local or off + nbytes <= self.nbytes, f"symmetric heap exhausted at {name}"
        self._offsets[name] = (off, nbytes)
        self._top = off + nbytes
        return off

    def ptr(self, name: str, rank: int, byte_offset: int = 0) -> int:
        return self.ptrs[rank] + self._offsets[name][0] + byte_offset

    def all_ptrs(self, name: str, byte_offset: int = 0) -> List[int]:
        return [self.ptr(name, r, byte_offset) for r in range(self.world)]

    def local_tensor(self, name: str, shape, dtype) -> torch.Tensor:
        return self._C.tensor_from_ptr(self.ptr(name, self.rank), list(shape), dtype, self.device.index or 0)

    def close(self) -> None:
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p:
                self._C.ipc_close(p)
        if self.local_ptr:
            self._C.ipc_free(self.local_ptr)
            self.local_ptr = 0
        self.ptrs = []
