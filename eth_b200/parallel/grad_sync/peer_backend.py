"""Peer-memory reduction backend of the gradient bucket executor.

The reduction of a bucket over its process group (data-parallel replicas and/or pipelines on one
NVSwitch node) is a two-shot all-reduce written for peer memory (`peer_reduce_pieces`,
csrc/comm.cu): rank r sums its 1 / W share of the bucket over all ranks with peer loads, in fp32
and in rank order (bit-identical results everywhere), and stores the sums into every rank's
buffer with peer stores, so both NVLink directions carry (W - 1) / W of the bucket. The reference
does pack -> NCCL all-reduce -> scale -> unpack (eth/runtime/megatron/grad_sync/executor.py:199-261).

Two layouts:
  direct  the stage's flat gradient buffer itself is a symmetric allocation, and the bucket's
          slices sit at the same offsets on every rank of the group (uniform layouts: pure data
          parallelism, or equal TP on all replicas). The kernel then works in place on the
          gradient buffers: no pack, no unpack, no scratch.
  packed  anything else (different TP widths between pipelines, replicated parameters with a
          contribution scale, evidence recording): pack into a symmetric scratch, reduce that
          scratch in place as one piece, unpack.

No kernel of this backend spins while it holds an SM's worth of resources: waiting for the peers'
"my gradients are final" and "my share is in your buffer" flags is done by `peer_flags`, a one-warp
kernel that fits beside a resident GEMM CTA. A rank that is early therefore cannot keep its own
(or, through a fused tensor-parallel GEMM, its partner's) compute kernels off the SMs, which is
what makes it safe to start reductions on a side stream while backward is still running.

Used when all ranks share one node; otherwise the executor falls back to the injected all-reduce.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ...ops import native
from ..peer_memory import SymmetricBuffer

_DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
FLAG_INTS_PER_GROUP = 64
FLAG_ARRIVE, FLAG_DONE = 0, 8     # csrc/comm.cuh: kFlagArrive, kFlagDone


def merge_pieces(pieces):
    """Coalesce (offset, rows, run, stride) pieces that are single runs lying back to back."""
    out: List[List[int]] = []
    for off, rows, run, stride in pieces:
        if out and rows == 1 and out[-1][1] == 1 and out[-1][0] + out[-1][2] == off:
            out[-1][2] += run
            out[-1][3] = out[-1][2]
        else:
            out.append([off, rows, run, stride if rows > 1 else run])
    return [tuple(p) for p in out]


class PeerReduceBackend:
    def __init__(self, plan, global_rank: int, coll, device, max_group: int = 8, grad_symm=None, grad_buf=None):
        self.max_group = max_group
        world = coll.world_size
        local_world = int(os.environ.get("LOCAL_WORLD_SIZE", world))
        if local_world != world:
            raise RuntimeError("peer-memory gradient reduction needs all ranks on one node")
        self.plan, self.rank, self.device, self.coll = plan, global_rank, torch.device(device), coll
        self.groups = {g.process_group_id: g.ranks for g in plan.process_groups}
        self.group_index = {g.process_group_id: i for i, g in enumerate(plan.process_groups)}
        self.world_ranks = tuple(range(world))
        # one scratch size for everybody: the largest bucket of any rank, per dtype
        self.max_numel = {}
        for (_r, dtype), numel in plan.max_scratch_numel_by_rank_and_dtype:
            self.max_numel[dtype] = max(self.max_numel.get(dtype, 0), numel)
        self.scratch: Dict[str, SymmetricBuffer] = {}
        self.flags = SymmetricBuffer(max(1, len(plan.process_groups)) * FLAG_INTS_PER_GROUP * 4, self.world_ranks,
                                     global_rank, None, self.device)
        self.epoch: Dict[int, int] = {}
        self.pending: Dict[int, int] = {}          # group index -> epoch whose done flags nobody has waited for yet
        self.grad_symm, self.grad_buf = grad_symm, grad_buf
        self.direct_tables: Dict[str, torch.Tensor] = {}
        self.packed_tables: Dict[str, torch.Tensor] = {}
        self.force_packed = False

    # ------------------------------------------------------------------ set-up
    def scratch_factory(self, name, numel, dtype, device):
        """Scratch of the executor: symmetric, sized by the largest bucket in the world (+ one vector
        of slack so that a bucket is reduced in whole 8-element vectors)."""
        n = max(self.max_numel.get(name, numel), numel) + 8
        esize = torch.empty((), dtype=dtype).element_size()
        buf = SymmetricBuffer(n * esize, self.world_ranks, self.rank, None, self.device)
        self.scratch[name] = buf
        return buf.tensor((n,), dtype)

    def attach(self, executor) -> None:
        """Decide per bucket whether the direct layout applies. Collective over the world: every rank
        publishes, per bucket, the pieces of its flat gradient buffer that make up the bucket; the
        direct layout is used where all ranks of the bucket's group published the same list."""
        mine = {}
        if self.grad_symm is not None and not self.force_packed:
            base, esize = self.grad_buf.data_ptr(), self.grad_buf.element_size()
            for b in executor.buckets:
                if not self.handles(b):
                    continue
                pieces, ok = [], True
                for view, _cursor, scale in executor._segments(b):
                    if scale != 1.0 or view.dtype != self.grad_buf.dtype:
                        ok = False
                        break
                    off = (view.data_ptr() - base) // esize
                    if view.dim() <= 1 or view.is_contiguous():
                        rows, run, stride = 1, view.numel(), view.numel()
                    else:
                        flat = view.reshape(-1, view.shape[-1]) if view.dim() > 2 else view
                        rows, run, stride = flat.shape[0], flat.shape[1], flat.stride(0)
                        if flat.stride(1) != 1 or flat.data_ptr() != view.data_ptr():
                            ok = False
                            break
                    if off < 0 or off % 8 or run % 8 or stride % 8 or off + (rows - 1) * stride + run > self.grad_buf.numel():
                        ok = False
                        break
                    pieces.append((off, rows, run, stride))
                if ok and pieces:
                    mine[b.bucket_id] = merge_pieces(pieces)
        everyone = [None] * len(self.world_ranks)
        self.coll.all_gather_object(everyone, mine)
        for b in executor.buckets:
            if b.bucket_id not in mine:
                continue
            ranks = self.groups[b.process_group_id]
            if all(everyone[r] is not None and everyone[r].get(b.bucket_id) == mine[b.bucket_id] for r in ranks):
                self.direct_tables[b.bucket_id] = torch.tensor(mine[b.bucket_id], dtype=torch.int64, device=self.device)

    def handles(self, bucket) -> bool:
        n = len(self.groups[bucket.process_group_id])
        return 1 < n <= self.max_group and bucket.grad_dtype in self.scratch

    def is_direct(self, bucket) -> bool:
        return bucket.bucket_id in self.direct_tables

    # ------------------------------------------------------------------ execution
    def _flag_ptrs(self, bucket):
        ranks = self.groups[bucket.process_group_id]
        gi = self.group_index[bucket.process_group_id]
        return ranks, gi, [self.flags.ptrs[r] + gi * FLAG_INTS_PER_GROUP * 4 for r in ranks]

    def _reduce(self, bucket, bases, table, dtype, scale):
        ranks, gi, flags = self._flag_ptrs(bucket)
        me = ranks.index(self.rank)
        epoch = self.epoch[gi] = self.epoch.get(gi, 0) + 1
        lib, status = native.lib(), native.status(self.device)
        # my gradients of this bucket are final (stream order); wait until that holds for every peer
        lib.peer_flags(flags, me, epoch, FLAG_ARRIVE, FLAG_ARRIVE, status)
        lib.peer_reduce_pieces(bases, flags, me, epoch, table, _DTYPE_CODE[dtype], float(scale))
        self.pending[gi] = epoch
        return flags, me, epoch, gi

    def reduce_direct(self, bucket, scale: float) -> None:
        """In-place two-shot all-reduce of the bucket's pieces of the flat gradient buffers. The
        result is complete on this rank only after `finish()`."""
        ranks = self.groups[bucket.process_group_id]
        bases = [self.grad_symm.ptrs[r] for r in ranks]
        self._reduce(bucket, bases, self.direct_tables[bucket.bucket_id], self.grad_buf.dtype, scale)

    def reduce_packed(self, bucket, payload, scale: float):
        """Two-shot all-reduce of the packed bucket inside the symmetric scratch; returns the scratch
        view holding the complete result (the peers' shares have been waited for)."""
        ranks = self.groups[bucket.process_group_id]
        buf = self.scratch[bucket.grad_dtype]
        n8 = (bucket.exact_numel + 7) // 8 * 8
        table = self.packed_tables.get(bucket.bucket_id)
        if table is None:
            table = torch.tensor([[0, 1, n8, n8]], dtype=torch.int64, device=self.device)
            self.packed_tables[bucket.bucket_id] = table
        flags, me, epoch, gi = self._reduce(bucket, [buf.ptrs[r] for r in ranks], table, payload.dtype, scale)
        native.lib().peer_flags(flags, me, epoch, -1, FLAG_DONE, native.status(self.device))
        self.pending.pop(gi, None)
        return payload

    def finish(self) -> None:
        """On the current stream: wait until every peer's share of every direct reduction issued so
        far has landed in this rank's gradient buffer (and the peers no longer read this rank's)."""
        if not self.pending:
            return
        lib, status = native.lib(), native.status(self.device)
        groups = {self.group_index[g.process_group_id]: g.ranks for g in self.plan.process_groups}
        for gi, epoch in sorted(self.pending.items()):
            ranks = groups[gi]
            flags = [self.flags.ptrs[r] + gi * FLAG_INTS_PER_GROUP * 4 for r in ranks]
            lib.peer_flags(flags, ranks.index(self.rank), epoch, -1, FLAG_DONE, status)
        self.pending.clear()
