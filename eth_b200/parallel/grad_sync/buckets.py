"""Bucket placement of canonical fragments and the deterministic process-group registry.

`tensor` mode: one bucket per fragment. `block` mode (block-wise all-reduce): consecutive
fragments with the same (process group, dtype, reduction) are concatenated until the byte cap;
a fragment is never split and an oversized fragment stands alone
(reference: eth/runtime/megatron/grad_sync/bucket_plan.py:115-152). The plan records, per rank,
the exact payload bytes and the largest bucket per dtype (the size of the persistent scratch),
and five hashes that all ranks compare before the first step.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Callable, Dict, Tuple

from .planner import CanonicalFragmentPlan, ProcessGroupSpec, _sort_key, stable_hash

DTYPE_BYTES = {"float16": 2, "bfloat16": 2, "float32": 4, "float64": 8}


def dtype_bytes(name: str) -> int:
    key = name[6:] if name.startswith("torch.") else name
    try:
        return DTYPE_BYTES[key]
    except KeyError as exc:
        raise ValueError(f"unsupported gradient dtype {name!r}") from exc


@dataclass(frozen=True)
class BucketFragmentPlacement:
    fragment_id: str
    destination_offset: int


@dataclass(frozen=True)
class CommunicationBucketSpec:
    bucket_id: str
    process_group_id: str
    grad_dtype: str
    reduction_semantics: str
    placements: Tuple[BucketFragmentPlacement, ...]
    exact_numel: int
    exact_bytes: int
    logical_region_begin: str
    logical_region_end: str
    semantic_hash: str
    oversized: bool


@dataclass(frozen=True)
class GradientSyncPlan:
    version: int
    sync_mode: str
    bucket_cap_bytes: int
    model_impl: str
    op_manifest_hash: str
    process_groups: Tuple[ProcessGroupSpec, ...]
    process_group_index_by_id: Tuple[Tuple[str, int], ...]
    canonical_fragments: tuple
    local_fragment_bindings_by_rank: tuple
    global_bucket_order: Tuple[CommunicationBucketSpec, ...]
    max_scratch_numel_by_rank_and_dtype: tuple
    exact_payload_bytes_by_rank: tuple
    padding_payload_bytes: int
    global_topology_hash: str
    global_manifest_hash: str
    global_fragment_hash: str
    global_plan_hash: str

    def buckets_for_rank(self, rank: int):
        ranks_of = {g.process_group_id: g.ranks for g in self.process_groups}
        return tuple(b for b in self.global_bucket_order if rank in ranks_of[b.process_group_id])

    def collective_count_for_rank(self, rank: int) -> int:
        return len(self.buckets_for_rank(rank))


def _close_bucket(frags, cap_bytes, groups) -> CommunicationBucketSpec:
    head = frags[0]
    width = dtype_bytes(head.grad_dtype)
    placements, cursor = [], 0
    for f in frags:
        placements.append(BucketFragmentPlacement(f.fragment_id, cursor))
        cursor += f.numel
    total_bytes = cursor * width
    digest = stable_hash({
        "version": 1, "process_group_id": head.process_group_id,
        "process_group_ranks": groups[head.process_group_id].ranks, "grad_dtype": head.grad_dtype,
        "reduction_semantics": head.reduction_semantics, "fragments": [asdict(f) for f in frags],
        "placements": [asdict(p) for p in placements], "exact_numel": cursor, "exact_bytes": total_bytes})
    return CommunicationBucketSpec(
        bucket_id="bucket-" + digest[:20], process_group_id=head.process_group_id,
        grad_dtype=head.grad_dtype, reduction_semantics=head.reduction_semantics,
        placements=tuple(placements), exact_numel=cursor, exact_bytes=total_bytes,
        logical_region_begin=head.logical_region_key, logical_region_end=frags[-1].logical_region_key,
        semantic_hash=digest, oversized=total_bytes > cap_bytes)


def bucketize(fragments, sync_mode: str, cap_bytes: int, groups) -> Tuple[CommunicationBucketSpec, ...]:
    if sync_mode not in ("tensor", "block"):
        raise ValueError(f"unsupported sync mode {sync_mode!r}")
    if cap_bytes <= 0:
        raise ValueError("bucket_cap_bytes must be positive")
    if sync_mode == "tensor":
        return tuple(_close_bucket((f,), cap_bytes, groups) for f in fragments)
    out, run, run_bytes, run_key = [], [], 0, None
    for f in fragments:
        size = f.numel * dtype_bytes(f.grad_dtype)
        key = (f.process_group_id, f.grad_dtype, f.reduction_semantics)
        if run and (key != run_key or run_bytes + size > cap_bytes):
            out.append(_close_bucket(tuple(run), cap_bytes, groups))
            run, run_bytes = [], 0
        run.append(f)
        run_bytes += size
        run_key = key
        if size > cap_bytes:  # oversized fragments stand alone
            out.append(_close_bucket(tuple(run), cap_bytes, groups))
            run, run_bytes, run_key = [], 0, None
    if run:
        out.append(_close_bucket(tuple(run), cap_bytes, groups))
    return tuple(out)


def build_gradient_sync_plan(fragment_plan: CanonicalFragmentPlan, sync_mode: str, bucket_cap_bytes: int,
                             model_impl: str, manifest_hash: str, topology_hash: str) -> GradientSyncPlan:
    groups = tuple(sorted(fragment_plan.process_groups, key=lambda g: g.ranks))
    by_id = {g.process_group_id: g for g in groups}
    index = {g.process_group_id: i for i, g in enumerate(groups)}
    frags = tuple(sorted(fragment_plan.fragments, key=lambda f: _sort_key(f.semantic_key)))
    dtype_rank = {d: i for i, d in enumerate(sorted({f.grad_dtype for f in frags}))}
    placement_order = tuple(sorted(
        frags, key=lambda f: (index[f.process_group_id], dtype_rank[f.grad_dtype], f.reduction_semantics,
                              _sort_key(f.semantic_key))))
    buckets = bucketize(placement_order, sync_mode, bucket_cap_bytes, by_id)
    payload: Dict[int, int] = {}
    scratch: Dict[tuple, int] = {}
    for b in buckets:
        for r in by_id[b.process_group_id].ranks:
            payload[r] = payload.get(r, 0) + b.exact_bytes
            scratch[(r, b.grad_dtype)] = max(scratch.get((r, b.grad_dtype), 0), b.exact_numel)
    bindings_payload = [(r, [asdict(x) for x in bs]) for r, bs in fragment_plan.local_bindings_by_rank]
    frag_hash = stable_hash({"canonical_fragments": [asdict(f) for f in frags],
                             "local_fragment_bindings_by_rank": bindings_payload})
    plan_hash = stable_hash({
        "version": 1, "sync_mode": sync_mode, "bucket_cap_bytes": bucket_cap_bytes, "model_impl": model_impl,
        "manifest_hash": manifest_hash, "topology_hash": topology_hash, "fragment_hash": frag_hash,
        "process_groups": [asdict(g) for g in groups], "canonical_fragments": [asdict(f) for f in frags],
        "local_fragment_bindings_by_rank": bindings_payload, "buckets": [asdict(b) for b in buckets]})
    return GradientSyncPlan(
        version=1, sync_mode=sync_mode, bucket_cap_bytes=bucket_cap_bytes, model_impl=model_impl,
        op_manifest_hash=manifest_hash, process_groups=groups,
        process_group_index_by_id=tuple((g.process_group_id, i) for i, g in enumerate(groups)),
        canonical_fragments=frags, local_fragment_bindings_by_rank=fragment_plan.local_bindings_by_rank,
        global_bucket_order=buckets, max_scratch_numel_by_rank_and_dtype=tuple(sorted(scratch.items())),
        exact_payload_bytes_by_rank=tuple(sorted(payload.items())), padding_payload_bytes=0,
        global_topology_hash=topology_hash, global_manifest_hash=manifest_hash,
        global_fragment_hash=frag_hash, global_plan_hash=plan_hash)


class ProcessGroupRegistry:
    """Creates every gradient-sync group exactly once, in one global order (sorted by ranks), on
    every rank -- the order `new_group` requires -- and freezes the table afterwards."""

    def __init__(self, process_groups, create_group: Callable[[Tuple[int, ...]], object]):
        self._specs = tuple(sorted(process_groups, key=lambda g: g.ranks))
        self._create = create_group
        self._handles: Dict[str, object] = {}
        self._created = 0

    def initialize(self) -> None:
        if self._handles:
            return
        ids, rank_sets = set(), set()
        for g in self._specs:
            if g.process_group_id in ids:
                raise ValueError(f"duplicate process group id {g.process_group_id}")
            if g.ranks in rank_sets:
                raise ValueError(f"duplicate process group ranks {g.ranks}")
            if g.ranks != tuple(sorted(set(g.ranks))):
                raise ValueError(f"process group ranks must be sorted and unique: {g.ranks}")
            ids.add(g.process_group_id)
            rank_sets.add(g.ranks)
            self._handles[g.process_group_id] = self._create(g.ranks)
            self._created += 1

    @property
    def group_count(self) -> int:
        return len(self._handles)

    @property
    def creation_count(self) -> int:
        return self._created

    def handle(self, process_group_id: str):
        if process_group_id not in self._handles:
            raise KeyError(f"process group {process_group_id} is not initialized")
        return self._handles[process_group_id]

    def ranks(self, process_group_id: str) -> Tuple[int, ...]:
        for g in self._specs:
            if g.process_group_id == process_group_id:
                return g.ranks
        raise KeyError(process_group_id)
