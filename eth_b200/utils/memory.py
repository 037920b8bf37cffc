"""Named, pre-allocated device buffers and ring buffers.

Long-running training wants its large temporaries allocated once: a `MemoryBuffer` hands out
zero-copy views of one allocation, a `RingMemBuffer` rotates over several so that a producer can
fill the next slot while a consumer still reads the previous one (reference:
eth/runtime/megatron/memory.py:24-145). `allocate_mem_buff` / `get_mem_buff` keep a process-wide
registry by name.
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch

_BUFFERS: Dict[str, "MemoryBuffer"] = {}


def allocate_mem_buff(name: str, numel: int, dtype: torch.dtype, track_usage: bool = False, device=None) -> "MemoryBuffer":
    if name in _BUFFERS:
        raise ValueError(f"memory buffer {name} already allocated")
    _BUFFERS[name] = MemoryBuffer(name, numel, dtype, track_usage, device)
    return _BUFFERS[name]


def get_mem_buff(name: str) -> "MemoryBuffer":
    return _BUFFERS[name]


def free_mem_buff(name: str) -> None:
    _BUFFERS.pop(name, None)


class MemoryBuffer:
    """One contiguous allocation; `add(tensor)` copies a tensor in and returns the view, `view(shape)`
    reserves space without copying. `reset()` starts over."""

    def __init__(self, name: str, numel: int, dtype: torch.dtype, track_usage: bool = False, device=None):
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.name, self.numel, self.dtype = name, int(numel), dtype
        self.data = torch.empty(self.numel, dtype=dtype, device=device, requires_grad=False)
        self._start = 0
        self.track_usage = track_usage
        self.in_use_value, self.total_value = 0.0, 0.0

    def reset(self) -> None:
        self._start = 0

    def is_in_use(self) -> bool:
        return self._start > 0

    def numel_in_use(self) -> int:
        return self._start

    def view(self, shape: Sequence[int]) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        end = self._start + n
        if end > self.numel:
            raise MemoryError(f"memory buffer {self.name}: {end} elements requested, {self.numel} available")
        out = self.data[self._start:end].view(*shape)
        self._start = end
        return out

    def add(self, tensor: torch.Tensor) -> torch.Tensor:
        if tensor.dtype != self.dtype:
            raise TypeError(f"memory buffer {self.name} holds {self.dtype}, got {tensor.dtype}")
        out = self.view(tensor.shape)
        out.copy_(tensor)
        return out

    def get_data(self) -> torch.Tensor:
        if self.track_usage:
            self.in_use_value += float(self._start)
            self.total_value += float(self.numel)
        return self.data[:self._start]

    def print_average_usage(self) -> None:
        if not self.track_usage:
            raise RuntimeError("usage tracking is off")
        print(f" > usage of {self.name} memory buffer: {100.0 * self.in_use_value / max(self.total_value, 1.0):.2f} %", flush=True)


class RingMemBuffer:
    """`num_buffers` memory buffers used round-robin."""

    def __init__(self, name: str, num_buffers: int, numel: int, dtype: torch.dtype, track_usage: bool = False, device=None):
        self.num_buffers = num_buffers
        self.buffers = [allocate_mem_buff(f"{name} {i}", numel, dtype, track_usage, device) for i in range(num_buffers)]
        self._index = -1

    def get_next_buffer(self) -> MemoryBuffer:
        nxt = (self._index + 1) % self.num_buffers
        buf = self.buffers[nxt]
        if buf.is_in_use():
            raise RuntimeError("ring buffer slot is still in use; reset() it before reuse")
        self._index = nxt
        return buf
