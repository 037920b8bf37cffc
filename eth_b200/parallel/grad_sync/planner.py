"""Canonical gradient fragments by interval arithmetic.

The same logical parameter can live under different tensor-parallel splits in different pipelines
and is replicated over each stage's data-parallel ranks (and, for a tied weight, over two stages).
Its gradient has to be summed over exactly the ranks that hold the same *elements*. The planner
works on the partition axis of each parameter:

  1. every holder contributes the global index spans it stores (`Span`: global [lo, hi) at a local
     offset; a strided shard has several);
  2. all span end points of all holders cut the axis into elementary intervals; inside one
     elementary interval every copy (pipeline, stage, data-parallel replica) has exactly one holder;
  3. elementary intervals with the same set of holder ranks are merged into one *fragment*: the
     unit that is reduced over one process group (the sorted holder ranks). Numbering the
     fragments of a parameter along the axis gives its canonical shard ids.

With nested TP widths this yields "shard k of the widest TP", the reference's canonical shards
(eth/runtime/megatron/grad_sync/planner.py:239-357); a narrower holder binds several fragments as
slices of its one tensor. Replicated parameters (LayerNorm, row-parallel biases) form one fragment
over all holders, each contributing grad / tp_degree because its TP peers hold identical copies
(:360-416). Of a tied weight only the root copy counts for the gradient norm (:419-440).

The plan is a pure, order-independent function of the gathered descriptors, so every rank
computes the same plan and ranks can compare its hash (:443-507).
"""
from __future__ import annotations

import bisect
import hashlib
import json
import math
from collections import defaultdict
from dataclasses import asdict, dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple


def stable_hash(value) -> str:
    blob = json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=True)
    return hashlib.sha256(blob.encode("utf-8")).hexdigest()


# ------------------------------------------------------------------------------------------
# plan records (field names are part of the dumped plan / evidence schema)
# ------------------------------------------------------------------------------------------
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
        return dict(self.local_bindings_by_rank).get(global_rank, ())

    def fragment(self, fragment_id: str) -> CanonicalGradientFragmentSpec:
        for f in self.fragments:
            if f.fragment_id == fragment_id:
                return f
        raise KeyError(fragment_id)


def group_id_for(ranks: Sequence[int]) -> str:
    return "pg-" + stable_hash({"ranks": tuple(ranks)})[:16]


def fragment_order(key):
    """Total order on semantic keys whose shard id may be None (replicated) or an int."""
    order_key, shard, regions = key
    return (tuple(order_key), -1 if shard is None else shard, tuple(regions))


_sort_key = fragment_order   # name used by the bucket planner


# ------------------------------------------------------------------------------------------
# spans: what a holder stores along the partition axis
# ------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Span:
    lo: int       # global start along the partition axis
    hi: int       # global end (exclusive)
    local: int    # offset of `lo` inside the holder's local tensor


def shard_spans(axis_size: int, degree: int, index: int, stride: int, what: str) -> Tuple[Span, ...]:
    """Spans of shard `index` of `degree`. With stride s the axis consists of s equal blocks and a
    shard stores its chunk of every block, one after the other."""
    pieces = degree * stride
    chunk, rest = divmod(axis_size, pieces)
    if rest:
        raise ValueError(f"nondivisible TP layout for {what}: axis of {axis_size} cannot be cut into "
                         f"{degree} shards x {stride} blocks")
    return tuple(Span((block * degree + index) * chunk, (block * degree + index + 1) * chunk, block * chunk)
                 for block in range(stride))


def shard_intervals(axis_size: int, degree: int, index: int, stride: int, what: str):
    """Global [lo, hi) ranges of a shard (the spans without their local offsets)."""
    return tuple((s.lo, s.hi) for s in shard_spans(axis_size, degree, index, stride, what))


class _Holder:
    """One rank's copy (or shard) of a logical parameter."""

    def __init__(self, desc, axis: int):
        self.desc, self.rank = desc, desc.global_rank
        self.copy = (desc.pipeline_id, desc.stage_id, desc.local_dp_rank)
        self.spans = shard_spans(desc.full_shape[axis], desc.local_tp_degree, desc.local_tp_rank,
                                 desc.partition_stride, desc.logical_param_id)
        self._starts = [s.lo for s in self.spans]

    def locate(self, lo: int, hi: int) -> Optional[int]:
        """Local offset of global [lo, hi) if one span contains it whole, else None."""
        i = bisect.bisect_right(self._starts, lo) - 1
        if i < 0:
            return None
        s = self.spans[i]
        return s.local + (lo - s.lo) if hi <= s.hi else None


# ------------------------------------------------------------------------------------------
# consistency of the holders of one parameter
# ------------------------------------------------------------------------------------------
# descriptor field -> what a disagreement between two holders is called
_MUST_AGREE = {
    "full_shape": "shape mismatch", "gradient_dtype": "dtype mismatch", "parameter_dtype": "dtype mismatch",
    "tensor_parallel": "replica semantics mismatch", "partition_stride": "stride mismatch",
    "model_impl": "model implementation mismatch", "op_manifest_hash": "manifest mismatch",
    "logical_region_key": "logical region mismatch", "semantic_order_key": "semantic order mismatch",
    "shared_weight_id": "shared weight mismatch", "shared_weight_root": "shared root mismatch",
}


def _partition_axis(desc) -> int:
    ndim = len(desc.full_shape)
    axis = desc.partition_dim + ndim if desc.partition_dim < 0 else desc.partition_dim
    if not 0 <= axis < ndim:
        raise ValueError(f"axis mismatch for {desc.logical_param_id}: partition_dim {desc.partition_dim} "
                         f"of a {ndim}-d tensor")
    return axis


def _check_own_coordinates(d) -> None:
    """A descriptor's group lists must be sorted, contain the rank, and match its coordinates."""
    lid, me = d.logical_param_id, d.global_rank
    for label, ranks, degree, coord in (("TP", tuple(d.local_tp_group_ranks), d.local_tp_degree, d.local_tp_rank),
                                        ("DP", tuple(d.local_dp_group_ranks), d.local_dp_degree, d.local_dp_rank)):
        if list(ranks) != sorted(ranks) or len(ranks) != degree:
            raise ValueError(f"{label} group mismatch for {lid} rank {me}")
        if me not in ranks or ranks.index(me) != coord:
            raise ValueError(f"{label} coordinate mismatch for {lid} rank {me}")
    if (d.local_cp_degree, d.local_cp_rank) != (1, 0):
        raise ValueError(f"CP coordinate mismatch for {lid} rank {me}")
    stage = tuple(d.stage_ranks)
    if list(stage) != sorted(stage) or me not in stage:
        raise ValueError(f"stage ranks mismatch for {lid} rank {me}")


def _check_agreement(logical_id: str, descs) -> None:
    first = descs[0]
    ranks_seen = set()
    for d in descs:
        if d.global_rank in ranks_seen:
            raise ValueError(f"duplicate owner rank {d.global_rank} for {logical_id}")
        ranks_seen.add(d.global_rank)
        for field, complaint in _MUST_AGREE.items():
            if getattr(d, field) == getattr(first, field):
                continue
            if field == "full_shape":
                who = ", ".join(f"rank={x.global_rank} full={x.full_shape} local={x.local_shape} "
                                f"tp={x.local_tp_rank}/{x.local_tp_degree}" for x in descs)
                raise ValueError(f"{complaint} for {logical_id}: {who}")
            raise ValueError(f"{complaint} for {logical_id}")
        _check_own_coordinates(d)


def _check_stage_grid(logical_id: str, descs) -> None:
    """Inside every (pipeline, stage) the holders must form a full TP x DP grid whose rows and
    columns are the groups the descriptors name."""
    stages = defaultdict(list)
    for d in descs:
        stages[(d.pipeline_id, d.stage_id)].append(d)
    for where, members in stages.items():
        tp, dp = members[0].local_tp_degree, members[0].local_dp_degree
        if any(d.local_dp_degree != dp for d in members):
            raise ValueError(f"DP degree mismatch for {logical_id} pipeline {where}")
        if any(d.local_tp_degree != tp for d in members):
            raise ValueError(f"TP degree mismatch for {logical_id} pipeline {where}")
        grid = {(d.local_dp_rank, d.local_tp_rank): d for d in members}
        if {dpr for dpr, _ in grid} != set(range(dp)):
            raise ValueError(f"missing owner DP replica for {logical_id} pipeline {where}")
        if len(grid) != len(members) or set(grid) != {(a, b) for a in range(dp) for b in range(tp)}:
            raise ValueError(f"missing owner TP rank for {logical_id} pipeline {where}")
        for dpr in range(dp):
            row = tuple(sorted(grid[(dpr, t)].global_rank for t in range(tp)))
            if any(tuple(grid[(dpr, t)].local_tp_group_ranks) != row for t in range(tp)):
                raise ValueError(f"TP group mismatch for {logical_id}")
        for t in range(tp):
            col = tuple(grid[(dpr, t)].global_rank for dpr in range(dp))
            if any(tuple(grid[(dpr, t)].local_dp_group_ranks) != col for dpr in range(dp)):
                raise ValueError(f"DP group mismatch for {logical_id} pipeline {where}")


def _check_tied_weights(by_id) -> None:
    families = defaultdict(list)
    for lid, descs in by_id.items():
        if descs[0].shared_weight_id is not None:
            families[descs[0].shared_weight_id].append((lid, descs[0]))
    same = ("full_shape", "parameter_dtype", "gradient_dtype", "tensor_parallel", "partition_dim", "partition_stride")
    for family, members in families.items():
        roots = [lid for lid, d in members if d.shared_weight_root]
        if len(roots) != 1:
            raise ValueError(f"shared root mismatch for {family}: expected one root, got {roots}")
        head = members[0][1]
        for lid, d in members[1:]:
            if any(getattr(d, f) != getattr(head, f) for f in same):
                raise ValueError(f"shared copy mismatch for {family} at {lid}")


# ------------------------------------------------------------------------------------------
# fragments of one parameter
# ------------------------------------------------------------------------------------------
def _numel(shape) -> int:
    return math.prod(shape) if shape else 1


def _make_fragment(logical_id, head, shard, ranks, regions, numel, reduction):
    group = group_id_for(ranks)
    key = (head.semantic_order_key, shard, regions)
    digest = stable_hash({"logical_param_id": logical_id, "canonical_shard_id": shard, "process_group_id": group,
                          "grad_dtype": head.gradient_dtype, "global_regions": regions, "semantic_key": key})
    counts = head.shared_weight_id is None or head.shared_weight_root
    return CanonicalGradientFragmentSpec(
        fragment_id="fragment-" + digest[:20], logical_param_id=logical_id, canonical_shard_id=shard,
        process_group_id=group, grad_dtype=head.gradient_dtype, reduction_semantics=reduction,
        logical_region_key=head.logical_region_key, global_regions=regions, numel=numel, semantic_key=key,
        optimizer_semantic_id=head.shared_weight_id or logical_id, include_in_optimizer_norm=counts,
        norm_owner_rank=min(ranks) if counts else None)


def _sharded_parameter(logical_id, descs):
    head = descs[0]
    axis = _partition_axis(head)
    if any(_partition_axis(d) != axis for d in descs):
        raise ValueError(f"axis mismatch for {logical_id}")
    size = head.full_shape[axis]
    row = _numel(head.full_shape) // size            # elements per index of the partition axis
    for d in descs:
        local = list(head.full_shape)
        local[axis] = size // d.local_tp_degree
        if size % d.local_tp_degree or tuple(d.local_shape) != tuple(local):
            raise ValueError(f"shape mismatch for {logical_id} rank {d.global_rank}")
    holders = [_Holder(d, axis) for d in descs]
    copies = defaultdict(list)
    for h in holders:
        copies[h.copy].append(h)
    # every copy must tile the axis exactly once
    for copy, members in copies.items():
        cursor = 0
        for s in sorted((s for h in members for s in h.spans), key=lambda s: s.lo):
            if s.lo != cursor:
                raise ValueError(f"local coverage overlap or gap for {logical_id} in copy {copy}")
            cursor = s.hi
        if cursor != size:
            raise ValueError(f"local coverage gap for {logical_id} in copy {copy}")
    cuts = sorted({p for h in holders for s in h.spans for p in (s.lo, s.hi)})
    # elementary interval -> the holder of every copy; merge intervals with equal holder sets
    merged: Dict[Tuple[int, ...], List[Tuple[int, int]]] = {}
    for lo, hi in zip(cuts, cuts[1:]):
        owners = []
        for copy in sorted(copies):
            hit = [h for h in copies[copy] if h.locate(lo, hi) is not None]
            if len(hit) != 1:
                raise ValueError(f"missing owner for {logical_id} indices [{lo}, {hi}) in copy {copy}")
            owners.append(hit[0].rank)
        ranks = tuple(sorted(owners))
        regions = merged.setdefault(ranks, [])
        if regions and regions[-1][1] == lo:
            regions[-1] = (regions[-1][0], hi)
        else:
            regions.append((lo, hi))
    by_rank = {h.rank: h for h in holders}
    groups, fragments, bindings = [], [], []
    for shard, (ranks, regions) in enumerate(sorted(merged.items(), key=lambda kv: kv[1][0])):
        regions = tuple(regions)
        frag = _make_fragment(logical_id, head, shard, ranks, regions, sum(hi - lo for lo, hi in regions) * row, "sum")
        groups.append(ProcessGroupSpec(frag.process_group_id, ranks, "gradient_sync"))
        fragments.append(frag)
        for r in ranks:
            h = by_rank[r]
            segments = tuple(TensorSegmentSpec(h.locate(lo, hi), hi - lo, tuple(h.desc.local_shape), lo, hi,
                                               (hi - lo) * row, axis) for lo, hi in regions)
            bindings.append(LocalFragmentBindingSpec(r, frag.fragment_id, logical_id, segments, 1.0))
    return groups, fragments, bindings


def _replicated_parameter(logical_id, descs):
    head = descs[0]
    for d in descs:
        if d.tp_replica_semantics != "identical_duplicate":
            raise ValueError(f"replica semantics invalid for {logical_id}")
        if tuple(d.local_shape) != tuple(d.full_shape):
            raise ValueError(f"shape mismatch for replicated {logical_id}")
    ranks = tuple(sorted(d.global_rank for d in descs))
    extent = head.full_shape[0] if head.full_shape else 1
    frag = _make_fragment(logical_id, head, None, ranks, ((0, extent),), _numel(head.full_shape),
                          "sum_identical_duplicates")
    bindings = []
    for d in sorted(descs, key=lambda x: x.global_rank):
        whole = TensorSegmentSpec(0, d.local_shape[0] if d.local_shape else 1, tuple(d.local_shape), 0, extent,
                                  _numel(d.local_shape), 0)
        # TP peers hold identical gradients of a replicated parameter: each brings 1 / tp of it
        bindings.append(LocalFragmentBindingSpec(d.global_rank, frag.fragment_id, logical_id, (whole,),
                                                 1.0 / d.local_tp_degree))
    return [ProcessGroupSpec(frag.process_group_id, ranks, "gradient_sync")], [frag], bindings


# ------------------------------------------------------------------------------------------
# the plan
# ------------------------------------------------------------------------------------------
def plan_canonical_fragments(descriptors: Iterable, expected_pipeline_ids: Iterable[int]) -> CanonicalFragmentPlan:
    descriptors = tuple(descriptors)
    pipelines = set(expected_pipeline_ids)
    if not pipelines:
        raise ValueError("expected_pipeline_ids must not be empty")
    for field, complaint in (("model_impl", "model implementation mismatch"), ("op_manifest_hash", "manifest mismatch")):
        if len({getattr(d, field) for d in descriptors}) > 1:
            raise ValueError(f"{complaint} across descriptors")
    index: Dict[str, list] = defaultdict(list)       # logical id -> holders
    for d in descriptors:
        if not d.requires_grad:
            raise ValueError(f"non-trainable descriptor {d.logical_param_id}")
        index[d.logical_param_id].append(d)
    for descs in index.values():
        descs.sort(key=lambda d: (d.pipeline_id, d.local_dp_rank, d.local_tp_rank, d.global_rank))
    _check_tied_weights(index)

    groups: Dict[str, ProcessGroupSpec] = {}
    fragments: List[CanonicalGradientFragmentSpec] = []
    bindings: List[LocalFragmentBindingSpec] = []
    for logical_id in sorted(index):
        descs = index[logical_id]
        absent = pipelines - {d.pipeline_id for d in descs}
        if absent or {d.pipeline_id for d in descs} - pipelines:
            raise ValueError(f"missing owner pipeline {sorted(absent)} for {logical_id}")
        _check_agreement(logical_id, descs)
        _check_stage_grid(logical_id, descs)
        build = _sharded_parameter if descs[0].tensor_parallel else _replicated_parameter
        g, f, b = build(logical_id, descs)
        for spec in g:
            known = groups.setdefault(spec.process_group_id, spec)
            if known.ranks != spec.ranks:
                raise ValueError(f"process group hash collision for {spec.ranks}")
        fragments += f
        bindings += b
    fragments.sort(key=lambda f: fragment_order(f.semantic_key))
    position = {f.fragment_id: i for i, f in enumerate(fragments)}
    per_rank = defaultdict(list)
    for b in bindings:
        per_rank[b.global_rank].append(b)
    frozen = tuple((r, tuple(sorted(per_rank[r], key=lambda b: position[b.fragment_id]))) for r in sorted(per_rank))
    return CanonicalFragmentPlan(
        process_groups=tuple(sorted(groups.values(), key=lambda g: g.ranks)), fragments=tuple(fragments),
        local_bindings_by_rank=frozen, fragment_hash=stable_hash([asdict(f) for f in fragments]))
