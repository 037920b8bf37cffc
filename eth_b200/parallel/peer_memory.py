"""Symmetric device buffers shared between the ranks of a group through CUDA IPC.

Every rank allocates the same sizes in the same order; the 64-byte IPC handles are exchanged with
an object all-gather over the (already initialised) process group, and each rank opens its peers'
handles, which maps their memory for loads and stores over NVLink. Kernels receive the list of
per-rank base pointers.
"""
from __future__ import annotations

import os
from typing import List, Sequence

import torch
import torch.distributed as dist

from ..ops import native


class SymmetricBuffer:
    """One symmetric allocation: `ptrs[i]` is the address of group-rank i's copy in this process."""

    def __init__(self, nbytes: int, group_ranks: Sequence[int], my_global_rank: int, group, device,
                 holds_data: bool = False):
        """`holds_data`: the buffer is a staging area that peers fill before it is read (not flags or
        counters, which must start at zero). With ETHB_POISON_STAGING=1 in the environment such a
        buffer starts as all-ones bytes, a NaN in every floating-point type, instead of zeros: a
        kernel that reads a slot before its producer wrote it then yields NaNs, which the overflow
        check of the optimizer and every numerics test catch, where stale zeros would pass silently.
        (A stand-in for an initcheck tool on memory that other GPUs write.)"""
        lib = native.lib()
        self.nbytes = int(nbytes)
        self.group_ranks = tuple(group_ranks)
        self.index = self.group_ranks.index(my_global_rank)
        self.device = torch.device(device)
        self.local_ptr, handle = lib.peer_alloc(self.nbytes)
        gathered = [None] * len(self.group_ranks)
        dist.all_gather_object(gathered, bytes(handle), group=group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for i, h in enumerate(gathered):
            if i == self.index:
                self.ptrs.append(self.local_ptr)
            else:
                p = lib.peer_open(h)
                self._opened.append(p)
                self.ptrs.append(p)
        if holds_data and os.environ.get("ETHB_POISON_STAGING", "0") == "1":
            import torch as _torch
            self.tensor((self.nbytes,), _torch.uint8).fill_(0xFF)
            _torch.cuda.synchronize(self.device)
        # nobody may touch a peer's buffer before everyone has mapped it
        dist.barrier(group=group)

    def tensor(self, shape, dtype, byte_offset: int = 0, index: int = None) -> torch.Tensor:
        i = self.index if index is None else index
        dev = self.device.index if self.device.index is not None else torch.cuda.current_device()
        return native.lib().tensor_from_ptr(self.ptrs[i] + byte_offset, list(shape), dtype, dev)

    def offset_ptrs(self, byte_offset: int) -> List[int]:
        return [p + byte_offset for p in self.ptrs]

    def close(self):
        lib = native.lib()
        for p in self._opened:
            try:
                lib.peer_close(p)
            except Exception:
                pass
        self._opened = []
