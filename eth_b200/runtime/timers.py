"""Named timers without host synchronisation on the hot path.

The reference's timers call `torch.cuda.synchronize()` on every start/stop when PROFILING=1, which
is its default (eth/runtime/megatron/global_vars.py:43, 203-220), so its pipeline transfers never
overlap compute. These timers record CUDA events on the current stream and resolve them lazily
when a report is requested; on CPU they fall back to wall-clock. Per-interval start/end stamps
(`--log-detail-compute-time`, :258-262, 320-331) are kept as event pairs as well.
"""
from __future__ import annotations

import time
from typing import Dict, List

import torch


class _Timer:
    def __init__(self, name: str, use_cuda: bool):
        self.name, self.use_cuda = name, use_cuda
        self._pairs: List[tuple] = []
        self._open = None
        self._elapsed_ms = 0.0
        self.count = 0

    def start(self):
        if self._open is not None:
            raise RuntimeError(f"timer {self.name} has already been started")
        if self.use_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open = ev
        else:
            self._open = time.perf_counter()

    def stop(self):
        if self._open is None:
            raise RuntimeError(f"timer {self.name} is not started")
        if self.use_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._pairs.append((self._open, ev))
        else:
            self._elapsed_ms += (time.perf_counter() - self._open) * 1e3
        self._open = None
        self.count += 1

    def _resolve(self):
        for a, b in self._pairs:
            b.synchronize()
            self._elapsed_ms += a.elapsed_time(b)
        self._pairs = []

    def elapsed(self, reset: bool = True) -> float:
        """Milliseconds accumulated so far."""
        running = self._open is not None
        if running:
            self.stop()
        self._resolve()
        out = self._elapsed_ms
        if reset:
            self._elapsed_ms, self.count = 0.0, 0
        if running:
            self.start()
        return out


class Timers:
    def __init__(self, use_cuda: bool = None):
        self.use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self.timers: Dict[str, _Timer] = {}

    def __call__(self, name: str) -> _Timer:
        if name not in self.timers:
            self.timers[name] = _Timer(name, self.use_cuda)
        return self.timers[name]

    def report(self, names=None, normalizer: float = 1.0, reset: bool = True) -> Dict[str, float]:
        names = names or sorted(self.timers)
        return {n: self.timers[n].elapsed(reset) / normalizer for n in names if n in self.timers}

    def log(self, names=None, normalizer: float = 1.0, reset: bool = True) -> str:
        rep = self.report(names, normalizer, reset)
        return "time (ms)" + "".join(f" | {n}: {v:.2f}" for n, v in rep.items())
