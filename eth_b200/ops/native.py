"""Loader of the native sm_100a library and of the per-device status word.

On a CUDA machine the compiled library must be present: ops raise instead of silently falling
back to PyTorch, so a missing build is noticed. On a CPU-only machine (unit tests, search,
validation CLIs) the library is optional and every op uses its PyTorch reference path.
"""
from __future__ import annotations

import importlib
import threading

import torch

_lock = threading.Lock()
_lib = None
_lib_error = None
_status = {}

STATUS_MESSAGES = {
    0: "ok",
    1: "timeout: MMA warp waited for a TMA stage",
    2: "timeout: TMA producer waited for a free stage",
    3: "timeout: epilogue waited for an accumulator",
    4: "timeout: MMA warp waited for a drained accumulator",
    5: "timeout: waited for a flag from a peer GPU",
    6: "timeout: waited for a flag from another CTA",
    7: "bad argument seen on the device",
}


def lib():
    """The compiled extension module (`eth_b200._C`). Raises if it cannot be imported."""
    global _lib, _lib_error
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            try:
                _lib = importlib.import_module("eth_b200._C")
            except Exception as exc:  # pragma: no cover - depends on the build
                _lib_error = exc
                raise RuntimeError(
                    "eth_b200 native library is not built; run `python -m eth_b200.build_ext`"
                ) from exc
    return _lib


def available() -> bool:
    try:
        lib()
        return True
    except RuntimeError:
        return False


def use_native(t: torch.Tensor) -> bool:
    """True when `t` must be processed by the CUDA kernels (and the library must exist)."""
    if not t.is_cuda:
        return False
    lib()
    return True


def status(device=None) -> torch.Tensor:
    """Per-device int32 status word that kernels write when a bounded wait expires."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = t
    return t


def check_status(device=None, reset: bool = True) -> None:
    """Synchronising read of the status word; raises with the recorded reason if non-zero."""
    t = status(device)
    code = int(t.item())
    if code != 0:
        if reset:
            t.zero_()
        raise RuntimeError(f"device kernel reported status {code}: {STATUS_MESSAGES.get(code, '?')}")


def launch_count() -> int:
    """Kernel launches issued by the native library since it was loaded."""
    return int(lib().launch_count()) if available() else 0
