"""Bucket placement of canonical fragments and the deterministic process-group registry.

A bucket is the unit of one gradient collective. Fragments are first put into *lanes*: everything
that may share a collective has the same (process group, gradient dtype, reduction kind). Inside a
lane, in semantic order,
  `tensor` mode cuts after every fragment (one collective per fragment), and
  `block` mode (block-wise all-reduce) cuts whenever the next fragment would push the running size
  over the byte cap; a fragment is never split, so one that alone exceeds the cap becomes a bucket
  of its own, flagged `oversized`
(reference behaviour: eth/runtime/megatron/grad_sync/bucket_plan.py:115-152). The plan also
records, per rank, the exact payload bytes and the largest bucket per dtype (the size of the
persistent scratch), and the hashes that all ranks compare before the first step (:155-241).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from itertools import groupby
from typing import Callable, Dict, Iterator, List, Sequence, Tuple

from .planner import CanonicalFragmentPlan, ProcessGroupSpec, fragment_order, stable_hash

SYNC_MODES = ("tensor", "block")
_ELEMENT_BYTES = {"float16": 2, "bfloat16": 2, "float32": 4, "float64": 8}


def dtype_bytes(name: str) -> int:
    short = name.split(".", 1)[1] if name.startswith("torch.") else name
    if short not in _ELEMENT_BYTES:
        raise ValueError(f"unsupported gradient dtype {name!r}")
    return _ELEMENT_BYTES[short]


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
        members = {g.process_group_id: g.ranks for g in self.process_groups}
        return tuple(b for b in self.global_bucket_order if rank in members[b.process_group_id])

    def collective_count_for_rank(self, rank: int) -> int:
        return len(self.buckets_for_rank(rank))


def _lane_of(fragment) -> tuple:
    return fragment.process_group_id, fragment.grad_dtype, fragment.reduction_semantics


def _cut_lane(fragments: Sequence, mode: str, cap_bytes: int) -> Iterator[List]:
    """Split one lane into runs of fragments, each run becoming a bucket."""
    run, used = [], 0
    for frag in fragments:
        size = frag.numel * dtype_bytes(frag.grad_dtype)
        if run and (mode == "tensor" or used + size > cap_bytes):
            yield run
            run, used = [], 0
        run.append(frag)
        used += size
    if run:
        yield run


def _seal(run, cap_bytes: int, group_ranks) -> CommunicationBucketSpec:
    first, last = run[0], run[-1]
    offsets, total = [], 0
    for frag in run:
        offsets.append(BucketFragmentPlacement(frag.fragment_id, total))
        total += frag.numel
    nbytes = total * dtype_bytes(first.grad_dtype)
    digest = stable_hash({
        "version": 1, "process_group_id": first.process_group_id, "process_group_ranks": group_ranks,
        "grad_dtype": first.grad_dtype, "reduction_semantics": first.reduction_semantics,
        "fragments": [asdict(f) for f in run], "placements": [asdict(p) for p in offsets],
        "exact_numel": total, "exact_bytes": nbytes})
    return CommunicationBucketSpec(
        bucket_id="bucket-" + digest[:20], process_group_id=first.process_group_id, grad_dtype=first.grad_dtype,
        reduction_semantics=first.reduction_semantics, placements=tuple(offsets), exact_numel=total,
        exact_bytes=nbytes, logical_region_begin=first.logical_region_key,
        logical_region_end=last.logical_region_key, semantic_hash=digest, oversized=nbytes > cap_bytes)


def bucketize(fragments, sync_mode: str, cap_bytes: int, groups) -> Tuple[CommunicationBucketSpec, ...]:
    """`fragments` must already be ordered so that the members of a lane are adjacent."""
    if sync_mode not in SYNC_MODES:
        raise ValueError(f"unsupported sync mode {sync_mode!r}")
    if cap_bytes <= 0:
        raise ValueError("bucket_cap_bytes must be positive")
    buckets = []
    for lane, members in groupby(fragments, key=_lane_of):
        for run in _cut_lane(list(members), sync_mode, cap_bytes):
            buckets.append(_seal(run, cap_bytes, groups[lane[0]].ranks))
    return tuple(buckets)


def build_gradient_sync_plan(fragment_plan: CanonicalFragmentPlan, sync_mode: str, bucket_cap_bytes: int,
                             model_impl: str, manifest_hash: str, topology_hash: str) -> GradientSyncPlan:
    groups = tuple(sorted(fragment_plan.process_groups, key=lambda g: g.ranks))
    group_by_id = {g.process_group_id: g for g in groups}
    group_pos = {g.process_group_id: i for i, g in enumerate(groups)}
    fragments = tuple(sorted(fragment_plan.fragments, key=lambda f: fragment_order(f.semantic_key)))
    dtype_pos = {name: i for i, name in enumerate(sorted({f.grad_dtype for f in fragments}))}
    laned = sorted(fragments, key=lambda f: (group_pos[f.process_group_id], dtype_pos[f.grad_dtype],
                                             f.reduction_semantics, fragment_order(f.semantic_key)))
    buckets = bucketize(laned, sync_mode, bucket_cap_bytes, group_by_id)

    payload_bytes: Dict[int, int] = {}
    scratch_numel: Dict[tuple, int] = {}
    for b in buckets:
        for rank in group_by_id[b.process_group_id].ranks:
            payload_bytes[rank] = payload_bytes.get(rank, 0) + b.exact_bytes
            slot = (rank, b.grad_dtype)
            scratch_numel[slot] = max(scratch_numel.get(slot, 0), b.exact_numel)

    bindings_blob = [(rank, [asdict(x) for x in bound]) for rank, bound in fragment_plan.local_bindings_by_rank]
    fragments_blob = [asdict(f) for f in fragments]
    fragment_hash = stable_hash({"canonical_fragments": fragments_blob,
                                 "local_fragment_bindings_by_rank": bindings_blob})
    plan_hash = stable_hash({
        "version": 1, "sync_mode": sync_mode, "bucket_cap_bytes": bucket_cap_bytes, "model_impl": model_impl,
        "manifest_hash": manifest_hash, "topology_hash": topology_hash, "fragment_hash": fragment_hash,
        "process_groups": [asdict(g) for g in groups], "canonical_fragments": fragments_blob,
        "local_fragment_bindings_by_rank": bindings_blob, "buckets": [asdict(b) for b in buckets]})
    return GradientSyncPlan(
        version=1, sync_mode=sync_mode, bucket_cap_bytes=bucket_cap_bytes, model_impl=model_impl,
        op_manifest_hash=manifest_hash, process_groups=groups,
        process_group_index_by_id=tuple(sorted(group_pos.items(), key=lambda kv: kv[1])),
        canonical_fragments=fragments, local_fragment_bindings_by_rank=fragment_plan.local_bindings_by_rank,
        global_bucket_order=buckets, max_scratch_numel_by_rank_and_dtype=tuple(sorted(scratch_numel.items())),
        exact_payload_bytes_by_rank=tuple(sorted(payload_bytes.items())), padding_payload_bytes=0,
        global_topology_hash=topology_hash, global_manifest_hash=manifest_hash,
        global_fragment_hash=fragment_hash, global_plan_hash=plan_hash)


class ProcessGroupRegistry:
    """Process groups of the plan, created once.

    `torch.distributed.new_group` must be called by every rank, for every group, in the same order;
    the registry walks the groups sorted by their rank tuples. After `initialize` the table is
    frozen: asking for an unknown id is an error, a second `initialize` does nothing."""

    def __init__(self, process_groups, create_group: Callable[[Tuple[int, ...]], object]):
        self._ranks_by_id = {}
        order = sorted(process_groups, key=lambda g: g.ranks)
        for g in order:
            if g.process_group_id in self._ranks_by_id:
                raise ValueError(f"duplicate process group id {g.process_group_id}")
            if list(g.ranks) != sorted(set(g.ranks)):
                raise ValueError(f"process group ranks must be sorted and unique: {g.ranks}")
            self._ranks_by_id[g.process_group_id] = g.ranks
        if len(set(self._ranks_by_id.values())) != len(self._ranks_by_id):
            raise ValueError("duplicate process group ranks in the plan")
        self._order = [g.process_group_id for g in order]
        self._make = create_group
        self._live: Dict[str, object] = {}
        self.creation_count = 0

    def initialize(self) -> None:
        if self._live:
            return
        for gid in self._order:
            self._live[gid] = self._make(self._ranks_by_id[gid])
            self.creation_count += 1

    @property
    def group_count(self) -> int:
        return len(self._live)

    def handle(self, process_group_id: str):
        try:
            return self._live[process_group_id]
        except KeyError:
            raise KeyError(f"process group {process_group_id} is not initialized") from None

    def ranks(self, process_group_id: str) -> Tuple[int, ...]:
        return self._ranks_by_id[process_group_id]
