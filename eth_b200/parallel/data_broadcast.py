"""Broadcast of a dict of tensors from the first rank of a tensor-parallel group to its peers.

Only one rank of a TP group needs to read a batch from the data loader; the others receive it
(reference: eth/runtime/megatron/mpu/data.py:76-117). Shapes travel first as one small int64
tensor, then all payloads as ONE flat tensor, so the cost is two collectives whatever the number
of keys.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch
import torch.distributed as dist

_MAX_DIMS = 5


def broadcast_data(keys: Sequence[str], data: Optional[Dict[str, torch.Tensor]], dtype: torch.dtype, src: int,
                   group=None, device=None) -> Dict[str, torch.Tensor]:
    """`data` is needed on rank `src` only (global rank); every rank returns the same dict."""
    rank = dist.get_rank()
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
    sizes = torch.zeros(len(keys) * _MAX_DIMS, dtype=torch.int64, device=device)
    if rank == src:
        for i, k in enumerate(keys):
            t = data[k]
            if t.dtype != dtype:
                raise TypeError(f"{k} has dtype {t.dtype}, expected {dtype}")
            if t.dim() > _MAX_DIMS:
                raise ValueError(f"{k} has more than {_MAX_DIMS} dimensions")
            for d, n in enumerate(t.shape):
                sizes[i * _MAX_DIMS + d] = n
    dist.broadcast(sizes, src, group=group)
    shapes, total = {}, 0
    host = sizes.tolist()
    for i, k in enumerate(keys):
        shape = [n for n in host[i * _MAX_DIMS:(i + 1) * _MAX_DIMS] if n > 0]
        shapes[k] = shape
        total += int(torch.Size(shape).numel())
    if rank == src:
        flat = torch.cat([data[k].reshape(-1).to(device) for k in keys])
    else:
        flat = torch.empty(total, dtype=dtype, device=device)
    dist.broadcast(flat, src, group=group)
    out, off = {}, 0
    for k in keys:
        n = int(torch.Size(shapes[k]).numel())
        out[k] = flat[off:off + n].view(shapes[k])
        off += n
    return out
