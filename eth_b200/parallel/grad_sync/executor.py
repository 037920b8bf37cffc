"""Execution of an immutable gradient-sync plan on one rank.

For every bucket this rank takes part in:  pack (gather the fragment slices of `main_grad` into
a persistent scratch, scaling replicated contributions) -> sum over the bucket's process group ->
multiply by the global normalisation scale -> unpack back into `main_grad`
(reference flow: eth/runtime/megatron/grad_sync/executor.py:199-261).

B200 specifics:
  * pack and unpack of a bucket are each ONE launch of a table-driven strided copy kernel
    (`strided_copy_scale`); the segment tables are built once and live on the device;
  * the reduction backend is injected. `collective` uses the given all-reduce callable (NCCL, or
    Gloo in CPU tests). `peer` runs the two-shot peer-memory kernel (`peer_reduce_pieces`, see
    peer_backend.py): where the bucket's slices sit at the same offsets of every rank's symmetric
    gradient buffer it works in place and pack / unpack disappear altogether.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Iterable, Optional

import torch

from . import runtime_evidence


def dtype_name(dtype) -> str:
    s = str(dtype)
    return s[6:] if s.startswith("torch.") else s


class GradientBucketExecutor:
    def __init__(self, plan, global_rank: int, local_descriptors: Iterable, local_runtime_bindings: Iterable,
                 process_group_registry, all_reduce_sum: Callable, runtime_evidence_dir: Optional[str] = None,
                 scratch_factory: Optional[Callable] = None, peer_backend=None):
        self.plan = plan
        self.global_rank = global_rank
        self._registry = process_group_registry
        self._all_reduce_sum = all_reduce_sum
        self._peer = peer_backend
        self._fragments = {f.fragment_id: f for f in plan.canonical_fragments}
        self._groups = {g.process_group_id: g for g in plan.process_groups}
        self._descriptors = self._index(local_descriptors, "descriptor")
        self._bindings = self._index(local_runtime_bindings, "runtime binding")
        self._specs = {b.fragment_id: b for r, bs in plan.local_fragment_bindings_by_rank if r == global_rank
                       for b in bs}
        self._my_buckets = tuple(b for b in plan.global_bucket_order
                                 if global_rank in self._groups[b.process_group_id].ranks)
        self._device = None
        self._validate()
        self._scratch = self._allocate_scratch(scratch_factory)
        self._tables: Dict[str, dict] = {}
        self.collectives_issued = 0
        self._evidence = (runtime_evidence.start_log(plan, global_rank, process_group_registry, self._scratch,
                                                     runtime_evidence_dir) if runtime_evidence_dir else None)
        if self._peer is not None and hasattr(self._peer, "attach"):
            self._peer.attach(self)

    # ------------------------------------------------------------------ set-up
    @staticmethod
    def _index(items, kind):
        out = {}
        for it in items:
            if it.logical_param_id in out:
                raise ValueError(f"duplicate {kind} for logical_param_id {it.logical_param_id}")
            out[it.logical_param_id] = it
        return out

    def _err(self, bucket, msg, binding=None):
        where = f"bucket {bucket.bucket_id} rank {self.global_rank}"
        if binding is not None:
            where += f" logical_param_id {binding.logical_param_id} fragment {binding.fragment_id}"
        return ValueError(f"{where}: {msg}")

    def _validate(self):
        devices = set()
        for bucket in self._my_buckets:
            for pl in bucket.placements:
                spec = self._specs.get(pl.fragment_id)
                if spec is None:
                    raise self._err(bucket, "missing local binding", self._fragments[pl.fragment_id])
                rt, desc = self._bindings.get(spec.logical_param_id), self._descriptors.get(spec.logical_param_id)
                if rt is None or desc is None:
                    raise self._err(bucket, "missing descriptor or main_grad binding", spec)
                if tuple(rt.main_grad.shape) != tuple(spec.source_segments[0].source_shape):
                    raise self._err(bucket, "main_grad shape mismatch", spec)
                if dtype_name(rt.main_grad.dtype) != dtype_name(bucket.grad_dtype):
                    raise self._err(bucket, "main_grad dtype mismatch", spec)
                if torch.device(rt.main_grad.device) != torch.device(rt.device):
                    raise self._err(bucket, "main_grad device mismatch", spec)
                devices.add(torch.device(rt.main_grad.device))
        if len(devices) > 1:
            raise ValueError(f"rank {self.global_rank} has multiple gradient execution devices: "
                             f"{sorted(map(str, devices))}")
        self._device = next(iter(devices), None)

    def _allocate_scratch(self, factory):
        want = {d: n for (r, d), n in self.plan.max_scratch_numel_by_rank_and_dtype if r == self.global_rank}
        if not want:
            return {}
        if self._device is None:
            raise ValueError(f"rank {self.global_rank} participates in gradient buckets without a device")
        by_name = {dtype_name(b.main_grad.dtype): b.main_grad.dtype for b in self._bindings.values()}
        out = {}
        for name, numel in want.items():
            dt = by_name.get(dtype_name(name))
            if dt is None:
                raise ValueError(f"rank {self.global_rank} has no main_grad with dtype {name}")
            if factory is not None:
                out[name] = factory(name, numel, dt, self._device)
            else:
                out[name] = torch.empty(numel, dtype=dt, device=self._device, requires_grad=False)
        return out

    @property
    def scratch_dtypes(self):
        return tuple(sorted(self._scratch))

    def scratch(self, name):
        return self._scratch[name]

    @property
    def buckets(self):
        return self._my_buckets

    # ------------------------------------------------------------------ slices
    def _view(self, spec, seg):
        rt, desc = self._bindings[spec.logical_param_id], self._descriptors[spec.logical_param_id]
        sharded = getattr(desc, "tensor_parallel", desc.partition_dim >= 0)
        if not sharded:
            if seg.flattened_numel != rt.main_grad.numel():
                raise ValueError(f"logical_param_id {spec.logical_param_id} replicated source numel mismatch")
            return rt.main_grad
        axis = desc.partition_dim + (len(rt.main_grad.shape) if desc.partition_dim < 0 else 0)
        if not 0 <= axis < len(rt.main_grad.shape):
            raise ValueError(f"logical_param_id {spec.logical_param_id} has invalid partition axis {desc.partition_dim}")
        if math.prod(seg.source_shape) != rt.main_grad.numel():
            raise ValueError(f"logical_param_id {spec.logical_param_id} source shape mismatch")
        return rt.main_grad.narrow(axis, seg.source_dim_offset, seg.source_dim_length)

    def _segments(self, bucket):
        """Yield (view, offset in bucket, contribution scale) for every local slice of the bucket."""
        for pl in bucket.placements:
            frag, spec = self._fragments[pl.fragment_id], self._specs[pl.fragment_id]
            cursor, seen = pl.destination_offset, 0
            for seg in spec.source_segments:
                view = self._view(spec, seg)
                if view.numel() != seg.flattened_numel:
                    raise self._err(bucket, "source segment numel mismatch", spec)
                if cursor + view.numel() > bucket.exact_numel:
                    raise self._err(bucket, "placement exceeds exact_numel", spec)
                yield view, cursor, spec.contribution_scale
                cursor += view.numel()
                seen += view.numel()
            if seen != frag.numel:
                raise self._err(bucket, f"packed {seen} elements, expected {frag.numel}", spec)

    def _table(self, bucket, payload):
        """Device-resident copy tables of a bucket (built on first use)."""
        key = (bucket.bucket_id, payload.data_ptr())
        tab = self._tables.get(key)
        if tab is not None:
            return tab
        pack_rows, unpack_rows, scales, biggest = [], [], set(), 1
        esize = payload.element_size()
        for view, off, scale in self._segments(bucket):
            if view.dim() <= 1 or view.is_contiguous():
                rows, run, stride = 1, view.numel(), view.numel()
            else:
                # a narrow() along the last axis of a 2-D tensor: `rows` runs of `run` elements
                flat = view.reshape(-1, view.shape[-1]) if view.dim() > 2 else view
                rows, run, stride = flat.shape[0], flat.shape[1], flat.stride(0)
                if flat.stride(1) != 1 or flat.data_ptr() != view.data_ptr():
                    raise ValueError("unsupported gradient slice layout")
            dst = payload.data_ptr() + off * esize
            pack_rows.append([view.data_ptr(), dst, rows, run, stride, run])
            unpack_rows.append([dst, view.data_ptr(), rows, run, run, stride])
            scales.add(scale)
            biggest = max(biggest, rows * run)
        if len(scales) > 1:
            raise ValueError(f"bucket {bucket.bucket_id} mixes contribution scales {sorted(scales)}")
        dev = payload.device
        tab = {"pack": torch.tensor(pack_rows, dtype=torch.int64, device=dev),
               "unpack": torch.tensor(unpack_rows, dtype=torch.int64, device=dev),
               "scale": scales.pop() if scales else 1.0, "max": biggest}
        self._tables[key] = tab
        return tab

    # ------------------------------------------------------------------ pack / unpack
    def pack(self, bucket, payload):
        if payload.is_cuda:
            from ...ops import native
            tab = self._table(bucket, payload)
            code = native.lib().strided_copy_scale
            dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[payload.dtype]
            code(tab["pack"], tab["max"], tab["scale"], dt, dt)
            return
        for view, off, scale in self._segments(bucket):
            dst = payload[off:off + view.numel()]
            dst.copy_(view.reshape(-1))
            if scale != 1.0:
                dst.mul_(scale)

    def unpack(self, bucket, payload, scale=1.0):
        if payload.is_cuda:
            from ...ops import native
            tab = self._table(bucket, payload)
            dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[payload.dtype]
            native.lib().strided_copy_scale(tab["unpack"], tab["max"], scale, dt, dt)
            return
        if scale != 1.0:
            payload.mul_(scale)
        for view, off, _ in self._segments(bucket):
            view.copy_(payload[off:off + view.numel()].view(view.shape))

    # ------------------------------------------------------------------ execution
    def execute_bucket(self, bucket, normalization_scale=1.0):
        if len(self._groups[bucket.process_group_id].ranks) == 1 and self._evidence is None:
            # nothing to reduce: only the normalisation applies, in place
            if normalization_scale != 1.0:
                for view, _off, _scale in self._segments(bucket):
                    view.mul_(normalization_scale)
            return
        if self._evidence is None and self._peer is not None and self._peer.is_direct(bucket):
            # in place on the symmetric gradient buffers: nothing to pack or unpack
            self._peer.reduce_direct(bucket, normalization_scale)
            self.collectives_issued += 1
            return
        payload = self._scratch[bucket.grad_dtype][:bucket.exact_numel]
        self.pack(bucket, payload)
        if self._evidence is not None:
            runtime_evidence.record_bucket(self._evidence, bucket, payload)
        if self._peer is not None and self._peer.handles(bucket):
            reduced = self._peer.reduce_packed(bucket, payload, normalization_scale)
            self.unpack(bucket, reduced, 1.0)
        else:
            self._all_reduce_sum(payload, self._registry.handle(bucket.process_group_id))
            self.unpack(bucket, payload, normalization_scale)
        self.collectives_issued += 1

    def bucket_first_op(self, bucket) -> int:
        """Smallest global op index among the parameters of a bucket: backward visits ops in decreasing
        index order, so once that op's backward has run every gradient of the bucket is final."""
        return min(self._descriptors[self._specs[pl.fragment_id].logical_param_id].global_op_index
                   for pl in bucket.placements)

    def needs_reduction(self, bucket) -> bool:
        return len(self._groups[bucket.process_group_id].ranks) > 1

    def uses_peer_backend(self, bucket) -> bool:
        return self._peer is not None and self._peer.handles(bucket)

    def execute(self, normalization_scale=1.0, skip=()):
        """Run all buckets of this rank in plan order, except those in `skip` (already reduced)."""
        if self._evidence is not None:
            runtime_evidence.open_iteration(self._evidence, normalization_scale)
        for bucket in self._my_buckets:
            if bucket.bucket_id not in skip:
                self.execute_bucket(bucket, normalization_scale)
        self.finish()
        if self._evidence is not None:
            runtime_evidence.close_iteration(self._evidence)
            runtime_evidence.write_report(self._evidence, self.plan)

    def finish(self) -> None:
        """Make the results of in-place peer reductions issued so far (on any stream the current one
        has joined) complete on the current stream."""
        if self._peer is not None:
            self._peer.finish()
