"""Canonical gradient fragments.

The same logical parameter can live under different tensor-parallel splits in different
pipelines (and be replicated over each stage's data-parallel ranks). A *canonical fragment* is the
finest shard of a logical parameter that some holder owns whole: with canonical TP degree
T = max TP over all holders, shard k of T along the partition axis. Every (pipeline, dp replica)
has exactly one rank that holds shard k -- possibly as a slice of a wider local tensor -- and the
sorted set of those ranks is the process group over which the fragment's gradient is summed.
Replicated parameters (LayerNorm, row-parallel biases) form one fragment over all holders, each
contributing grad / local_tp_degree because its TP peers hold identical duplicates.

Planning is deterministic and purely a function of the gathered descriptors, so every rank
computes the same plan and can compare hashes (reference behaviour:
eth/runtime/megatron/grad_sync/planner.py:239-357 sharded, :360-416 replicated, :419-440 tied
weights, :443-507 ordering and hash).
"""
from __future__ import annotations

import hashlib
import json
import math
from dataclasses import asdict, dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple


def stable_hash(value) -> str:
    blob = json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=True)
    return hashlib.sha256(blob.encode("utf-8")).hexdigest()


@dataclass(frozen=True)
class TensorSegmentSpec:
    """`source_dim_length` consecutive indices starting at `source_dim_offset` along the partition
    axis of a local tensor of shape `source_shape`; they are global coordinates [begin, end)."""
    source_dim_offset: int
    source_dim_length: int
    source_shape: Tuple[int, ...]
    global_coordinate_begin: int
    global_coordinate_end: int
    flattened_numel: int
    axis: int = 0


@dataclass(frozen=True)
class ProcessGroupSpec:
    process_group_id: str
    ranks: Tuple[int, ...]
    semantic_kind: str


@dataclass(frozen=True)
class CanonicalGradientFragmentSpec:
    fragment_id: str
    logical_param_id: str
    canonical_shard_id: Optional[int]
    process_group_id: str
    grad_dtype: str
    reduction_semantics: str           # "sum" | "sum_identical_duplicates"
    logical_region_key: str
    global_regions: Tuple[Tuple[int, int], ...]
    numel: int
    semantic_key: tuple
    optimizer_semantic_id: str
    include_in_optimizer_norm: bool
    norm_owner_rank: Optional[int]


@dataclass(frozen=True)
class LocalFragmentBindingSpec:
    global_rank: int
    fragment_id: str
    logical_param_id: str
    source_segments: Tuple[TensorSegmentSpec, ...]
    contribution_scale: float


@dataclass(frozen=True)
class CanonicalFragmentPlan:
    process_groups: Tuple[ProcessGroupSpec, ...]
    fragments: Tuple[CanonicalGradientFragmentSpec, ...]
    local_bindings_by_rank: Tuple[Tuple[int, Tuple[LocalFragmentBindingSpec, ...]], ...]
    fragment_hash: str

    def bindings_for_rank(self, global_rank: int) -> Tuple[LocalFragmentBindingSpec, ...]:
        for rank, bindings in self.local_bindings_by_rank:
            if rank == global_rank:
                return bindings
        return ()

    def fragment(self, fragment_id: str) -> CanonicalGradientFragmentSpec:
        for f in self.fragments:
            if f.fragment_id == fragment_id:
                return f
        raise KeyError(fragment_id)


def group_id_for(ranks: Sequence[int]) -> str:
    return "pg-" + stable_hash({"ranks": tuple(ranks)})[:16]


def _numel(shape) -> int:
    return math.prod(shape) if shape else 1


def _axis(desc) -> int:
    ax = desc.partition_dim
    if ax < 0:
        ax += len(desc.full_shape)
    if not 0 <= ax < len(desc.full_shape):
        raise ValueError(f"axis mismatch for {desc.logical_param_id}: {desc.partition_dim}")
    return ax


def shard_intervals(axis_size: int, degree: int, index: int, stride: int, what: str):
    """Global index ranges owned by shard `index` of `degree`. With stride s the axis is cut into
    s blocks and each shard owns one chunk of every block (fused QKV / gated layouts)."""
    div = degree * stride
    if axis_size % div:
        raise ValueError(f"nondivisible TP layout for {what}: axis {axis_size}, TP {degree}, stride {stride}")
    chunk = axis_size // div
    return tuple(((b * degree + index) * chunk, (b * degree + index + 1) * chunk) for b in range(stride))


def _locate(desc, regions, axis) -> Tuple[TensorSegmentSpec, ...]:
    """Where `regions` (global) sit inside `desc`'s local tensor, or () if not fully contained."""
    mine = shard_intervals(desc.full_shape[axis], desc.local_tp_degree, desc.local_tp_rank,
                           desc.partition_stride, desc.logical_param_id)
    other = _numel(desc.full_shape) // desc.full_shape[axis]
    found: List[TensorSegmentSpec] = []
    local_off = 0
    for lo, hi in mine:
        for rb, re in regions:
            b, e = max(lo, rb), min(hi, re)
            if b < e:
                found.append(TensorSegmentSpec(local_off + b - lo, e - b, tuple(desc.local_shape), b, e,
                                               (e - b) * other, axis))
        local_off += hi - lo
    if tuple((s.global_coordinate_begin, s.global_coordinate_end) for s in found) != tuple(regions):
        return ()
    return tuple(found)


_SAME_EVERYWHERE = (
    ("full_shape", "shape mismatch"), ("gradient_dtype", "dtype mismatch"),
    ("parameter_dtype", "dtype mismatch"), ("tensor_parallel", "replica semantics mismatch"),
    ("partition_stride", "stride mismatch"), ("model_impl", "model implementation mismatch"),
    ("op_manifest_hash", "manifest mismatch"), ("logical_region_key", "logical region mismatch"),
    ("semantic_order_key", "semantic order mismatch"), ("shared_weight_id", "shared weight mismatch"),
    ("shared_weight_root", "shared root mismatch"),
)


def _check_holders(logical_id: str, descs) -> Dict[tuple, Dict[int, list]]:
    """Consistency of all holders of one logical parameter.

    Returns {(pipeline, stage): {dp_rank: [descs]}}. One logical parameter normally lives in one
    stage per pipeline; a tied weight (the word embedding, used by the first stage's embedding and
    by the last stage's output head) lives in two, and both copies join the same fragment groups,
    so one all-reduce sums embedding-side and head-side gradients of all pipelines and replicas."""
    ref = descs[0]
    seen = set()
    for d in descs:
        if d.global_rank in seen:
            raise ValueError(f"duplicate owner rank {d.global_rank} for {logical_id}")
        seen.add(d.global_rank)
        for field, msg in _SAME_EVERYWHERE:
            if getattr(d, field) != getattr(ref, field):
                if field == "full_shape":
                    detail = ", ".join(
                        f"rank={x.global_rank} full={x.full_shape} local={x.local_shape} "
                        f"tp={x.local_tp_rank}/{x.local_tp_degree}" for x in descs)
                    raise ValueError(f"{msg} for {logical_id}: {detail}")
                raise ValueError(f"{msg} for {logical_id}")
        if d.tensor_parallel and _axis(d) != _axis(ref):
            raise ValueError(f"axis mismatch for {logical_id}")
        for label, ranks, degree, coord in (("TP", d.local_tp_group_ranks, d.local_tp_degree, d.local_tp_rank),
                                            ("DP", d.local_dp_group_ranks, d.local_dp_degree, d.local_dp_rank)):
            ranks = tuple(ranks)
            if tuple(sorted(ranks)) != ranks or len(ranks) != degree:
                raise ValueError(f"{label} group mismatch for {logical_id} rank {d.global_rank}")
            if d.global_rank not in ranks or ranks.index(d.global_rank) != coord:
                raise ValueError(f"{label} coordinate mismatch for {logical_id} rank {d.global_rank}")
        if d.local_cp_degree != 1 or d.local_cp_rank != 0:
            raise ValueError(f"CP coordinate mismatch for {logical_id} rank {d.global_rank}")
        sr = tuple(d.stage_ranks)
        if tuple(sorted(sr)) != sr or d.global_rank not in sr:
            raise ValueError(f"stage ranks mismatch for {logical_id} rank {d.global_rank}")
    by_pipe: Dict[tuple, Dict[int, list]] = {}
    for d in descs:
        by_pipe.setdefault((d.pipeline_id, d.stage_id), {}).setdefault(d.local_dp_rank, []).append(d)
    for pid, replicas in by_pipe.items():
        members = [d for d in descs if (d.pipeline_id, d.stage_id) == pid]
        dp = members[0].local_dp_degree
        if any(d.local_dp_degree != dp for d in members):
            raise ValueError(f"DP degree mismatch for {logical_id} pipeline {pid}")
        if set(replicas) != set(range(dp)):
            raise ValueError(f"missing owner DP replica for {logical_id} pipeline {pid}")
        tp = members[0].local_tp_degree
        if any(d.local_tp_degree != tp for d in members):
            raise ValueError(f"TP degree mismatch for {logical_id} pipeline {pid}")
        for dpr, holders in replicas.items():
            if len(holders) != tp or {d.local_tp_rank for d in holders} != set(range(tp)):
                raise ValueError(f"missing owner TP rank for {logical_id} pipeline {pid} DP {dpr}")
            group = tuple(sorted(d.global_rank for d in holders))
            if any(tuple(d.local_tp_group_ranks) != group for d in holders):
                raise ValueError(f"TP group mismatch for {logical_id}")
        for t in range(tp):
            lane = sorted((d for hs in replicas.values() for d in hs if d.local_tp_rank == t),
                          key=lambda d: d.local_dp_rank)
            group = tuple(d.global_rank for d in lane)
            if any(tuple(d.local_dp_group_ranks) != group for d in lane):
                raise ValueError(f"DP group mismatch for {logical_id} pipeline {pid}")
    return by_pipe


def _fragment(logical_id, ref, shard, group_ranks, regions, numel, reduction):
    pgid = group_id_for(group_ranks)
    order_key = (ref.semantic_order_key, shard, regions)
    fid = "fragment-" + stable_hash({
        "logical_param_id": logical_id, "canonical_shard_id": shard, "process_group_id": pgid,
        "grad_dtype": ref.gradient_dtype, "global_regions": regions, "semantic_key": order_key})[:20]
    in_norm = ref.shared_weight_id is None or ref.shared_weight_root
    return CanonicalGradientFragmentSpec(
        fragment_id=fid, logical_param_id=logical_id, canonical_shard_id=shard, process_group_id=pgid,
        grad_dtype=ref.gradient_dtype, reduction_semantics=reduction,
        logical_region_key=ref.logical_region_key, global_regions=regions, numel=numel,
        semantic_key=order_key, optimizer_semantic_id=ref.shared_weight_id or logical_id,
        include_in_optimizer_norm=in_norm, norm_owner_rank=min(group_ranks) if in_norm else None)


def _plan_sharded(logical_id, descs, by_pipe):
    ref = descs[0]
    axis = _axis(ref)
    canon = max(d.local_tp_degree for d in descs)
    shard_intervals(ref.full_shape[axis], canon, 0, ref.partition_stride, logical_id)
    for d in descs:
        if canon % d.local_tp_degree:
            raise ValueError(f"nondivisible canonical TP degree for {logical_id}: {canon} % {d.local_tp_degree}")
        want = list(ref.full_shape)
        want[axis] //= d.local_tp_degree
        if tuple(d.local_shape) != tuple(want):
            raise ValueError(f"shape mismatch for {logical_id} rank {d.global_rank}")
    other = _numel(ref.full_shape) // ref.full_shape[axis]
    groups, frags, binds = [], [], []
    for shard in range(canon):
        regions = shard_intervals(ref.full_shape[axis], canon, shard, ref.partition_stride, logical_id)
        owners = []
        for pid in sorted(by_pipe):
            for dpr in sorted(by_pipe[pid]):
                hits = [(d, seg) for d in by_pipe[pid][dpr] for seg in [_locate(d, regions, axis)] if seg]
                if len(hits) != 1:
                    raise ValueError(f"missing owner for {logical_id} shard {shard} pipeline {pid} DP {dpr}")
                owners.append(hits[0])
        ranks = tuple(sorted(d.global_rank for d, _ in owners))
        frag = _fragment(logical_id, ref, shard, ranks, regions,
                         sum(e - b for b, e in regions) * other, "sum")
        groups.append(ProcessGroupSpec(frag.process_group_id, ranks, "gradient_sync"))
        frags.append(frag)
        for d, segs in owners:
            binds.append(LocalFragmentBindingSpec(d.global_rank, frag.fragment_id, logical_id, segs, 1.0))
    # every local element must be bound exactly once
    for d in descs:
        spans = sorted((s.source_dim_offset, s.source_dim_offset + s.source_dim_length)
                       for b in binds if b.global_rank == d.global_rank for s in b.source_segments)
        cursor = 0
        for b, e in spans:
            if b != cursor or e <= b:
                raise ValueError(f"local coverage overlap or gap for {logical_id} rank {d.global_rank}")
            cursor = e
        if cursor != d.local_shape[axis]:
            raise ValueError(f"local coverage gap for {logical_id} rank {d.global_rank}")
    return groups, frags, binds


def _plan_replicated(logical_id, descs):
    ref = descs[0]
    for d in descs:
        if d.tp_replica_semantics != "identical_duplicate":
            raise ValueError(f"replica semantics invalid for {logical_id}")
        if tuple(d.local_shape) != tuple(d.full_shape):
            raise ValueError(f"shape mismatch for replicated {logical_id}")
    ranks = tuple(sorted(d.global_rank for d in descs))
    first = ref.full_shape[0] if ref.full_shape else 1
    regions = ((0, first),)
    frag = _fragment(logical_id, ref, None, ranks, regions, _numel(ref.full_shape),
                     "sum_identical_duplicates")
    binds = []
    for d in sorted(descs, key=lambda x: x.global_rank):
        seg = TensorSegmentSpec(0, d.local_shape[0] if d.local_shape else 1, tuple(d.local_shape), 0, first,
                                _numel(d.local_shape), 0)
        binds.append(LocalFragmentBindingSpec(d.global_rank, frag.fragment_id, logical_id, (seg,),
                                              1.0 / d.local_tp_degree))
    return [ProcessGroupSpec(frag.process_group_id, ranks, "gradient_sync")], [frag], binds


def _check_tied(by_id) -> None:
    tied: Dict[str, list] = {}
    for lid, descs in by_id.items():
        if descs[0].shared_weight_id is not None:
            tied.setdefault(descs[0].shared_weight_id, []).append((lid, descs))
    for sid, members in tied.items():
        roots = [lid for lid, descs in members if descs[0].shared_weight_root]
        if len(roots) != 1:
            raise ValueError(f"shared root mismatch for {sid}: expected one root, got {roots}")
        ref = members[0][1][0]
        for lid, descs in members[1:]:
            for field in ("full_shape", "parameter_dtype", "gradient_dtype", "tensor_parallel",
                          "partition_dim", "partition_stride"):
                if getattr(descs[0], field) != getattr(ref, field):
                    raise ValueError(f"shared copy mismatch for {sid} at {lid}")


def plan_canonical_fragments(descriptors: Iterable, expected_pipeline_ids: Iterable[int]) -> CanonicalFragmentPlan:
    descriptors = tuple(descriptors)
    if len({d.model_impl for d in descriptors}) > 1:
        raise ValueError("model implementation mismatch across descriptors")
    if len({d.op_manifest_hash for d in descriptors}) > 1:
        raise ValueError("manifest mismatch across descriptors")
    by_id: Dict[str, list] = {}
    for d in descriptors:
        if not d.requires_grad:
            raise ValueError(f"non-trainable descriptor {d.logical_param_id}")
        by_id.setdefault(d.logical_param_id, []).append(d)
    want_pipes = set(expected_pipeline_ids)
    if not want_pipes:
        raise ValueError("expected_pipeline_ids must not be empty")
    _check_tied(by_id)
    groups: Dict[str, ProcessGroupSpec] = {}
    frags: List[CanonicalGradientFragmentSpec] = []
    binds: List[LocalFragmentBindingSpec] = []
    for lid in sorted(by_id):
        descs = sorted(by_id[lid], key=lambda d: (d.pipeline_id, d.local_dp_rank, d.local_tp_rank, d.global_rank))
        have = {d.pipeline_id for d in descs}
        if have != want_pipes:
            raise ValueError(f"missing owner pipeline {sorted(want_pipes - have)} for {lid}")
        by_pipe = _check_holders(lid, descs)
        g, f, b = _plan_sharded(lid, descs, by_pipe) if descs[0].tensor_parallel else _plan_replicated(lid, descs)
        for item in g:
            old = groups.get(item.process_group_id)
            if old is not None and old.ranks != item.ranks:
                raise ValueError(f"process group hash collision for {item.ranks}")
            groups[item.process_group_id] = item
        frags.extend(f)
        binds.extend(b)
    frags.sort(key=lambda f: _sort_key(f.semantic_key))
    order = {f.fragment_id: i for i, f in enumerate(frags)}
    per_rank: Dict[int, list] = {}
    for b in binds:
        per_rank.setdefault(b.global_rank, []).append(b)
    frozen = tuple((r, tuple(sorted(bs, key=lambda b: order[b.fragment_id]))) for r, bs in sorted(per_rank.items()))
    return CanonicalFragmentPlan(
        process_groups=tuple(sorted(groups.values(), key=lambda g: g.ranks)),
        fragments=tuple(frags), local_bindings_by_rank=frozen,
        fragment_hash=stable_hash([asdict(f) for f in frags]))


def _sort_key(key):
    """Total order on semantic keys whose shard id may be None (replicated) or an int."""
    order_key, shard, regions = key
    return (tuple(order_key), -1 if shard is None else shard, tuple(regions))
