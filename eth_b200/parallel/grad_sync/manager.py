"""Bring-up of canonical gradient synchronisation on one rank, and the handle the engine keeps.

Bring-up is a fixed sequence of stages, each of which ends in an agreement between ranks:

    descriptors   every rank learns every rank's parameter descriptors     (world gather)
    plan          fragments + buckets, computed locally from the same input
    plan hash     all ranks must have computed the same plan               (world gather)
    groups        every process group created once, in one global order
    manifests     the members of each group compare their bucket lists     (group gather)
    runtime       executor (+ optional peer-memory backend) and optimizer semantics

Collectives are passed in as callables, so the sequence runs unchanged under in-memory fakes in
unit tests, over Gloo in multi-process CPU tests and over NCCL in training
(reference: eth/runtime/megatron/grad_sync/manager.py:122-214).
"""
from __future__ import annotations

import json
from dataclasses import asdict
from pathlib import Path
from typing import Callable, Sequence

from .buckets import ProcessGroupRegistry, build_gradient_sync_plan
from .executor import GradientBucketExecutor
from .optimizer_semantics import CanonicalOptimizerSemantics
from .planner import plan_canonical_fragments


def dump_gradient_sync_plan(plan, path) -> None:
    target = Path(path)
    target.parent.mkdir(parents=True, exist_ok=True)
    target.write_text(json.dumps(asdict(plan), indent=2, sort_keys=True) + "\n", encoding="utf-8")


def require_agreement(mine, gather: Callable[[list, object], None], peers: int, complaint: str):
    """Gather `mine` from `peers` ranks and insist that all of them sent the same value."""
    seen = [None] * peers
    gather(seen, mine)
    if any(other != mine for other in seen):
        raise ValueError(f"{complaint}: {tuple(seen)}")
    return seen


def bucket_manifest(plan, process_group_id: str) -> tuple:
    """What the members of a group compare: the group's buckets as (hash, numel, dtype, #fragments)."""
    return tuple((b.semantic_hash, b.exact_numel, b.grad_dtype, len(b.placements))
                 for b in plan.global_bucket_order if b.process_group_id == process_group_id)


class GradientSyncManager:
    """Plan, process groups, bucket executor and optimizer semantics of one rank."""

    def __init__(self, plan, registry: ProcessGroupRegistry, executor: GradientBucketExecutor,
                 optimizer_semantics: CanonicalOptimizerSemantics):
        self.plan, self.registry, self.executor, self.optimizer_semantics = plan, registry, executor, optimizer_semantics

    def execute(self, normalization_scale=1.0):
        self.executor.execute(normalization_scale=normalization_scale)

    def my_groups(self):
        me = self.optimizer_semantics.global_rank
        return [g for g in self.plan.process_groups if me in g.ranks]

    def _on_group(self, broadcast):
        """Adapter: the semantics layer names a group by id, `broadcast` wants the live handle."""
        def call(payload, source_rank, process_group_id, *_unused):
            broadcast(payload, source_rank, self.registry.handle(process_group_id))
        return call

    def synchronize_parameters(self, broadcast):
        self.optimizer_semantics.synchronize_parameters(self._on_group(broadcast))

    def synchronize_shared_root_gradients(self, broadcast):
        self.optimizer_semantics.synchronize_shared_root_gradients(self._on_group(broadcast))

    def synchronize_optimizer_state(self, optimizer, broadcast, all_gather_group_object):
        sem, view = self.optimizer_semantics, optimizer.state_for_model_parameter
        for group in self.my_groups():
            handle = self.registry.handle(group.process_group_id)
            require_agreement(sem.optimizer_state_manifest_for_group(group.process_group_id, view),
                              lambda out, obj, h=handle: all_gather_group_object(out, obj, h), len(group.ranks),
                              f"optimizer state manifest mismatch for process group {group.process_group_id}")
        sem.synchronize_optimizer_state(view, self._on_group(broadcast))


def initialize_gradient_sync(*, local_descriptors: Sequence, local_runtime_bindings: Sequence, topology, model_impl,
                             manifest_hash, sync_mode, bucket_cap_bytes, global_rank, all_gather_object,
                             all_gather_group_object, create_group, all_reduce_sum, control_device="cpu",
                             runtime_evidence_dir=None, scratch_factory=None, peer_backend_factory=None):
    world = topology.world_size
    # -- descriptors
    per_rank = [None] * world
    all_gather_object(per_rank, tuple(local_descriptors))
    if None in per_rank:
        raise ValueError("gradient metadata gather returned an incomplete world")
    # -- plan (a pure function of the gathered descriptors)
    fragments = plan_canonical_fragments([d for rank_descs in per_rank for d in rank_descs],
                                         expected_pipeline_ids=topology.pipeline_ids)
    plan = build_gradient_sync_plan(fragments, sync_mode, bucket_cap_bytes, model_impl, manifest_hash,
                                    topology.fingerprint)
    # -- plan hash
    require_agreement(plan.global_plan_hash, all_gather_object, world, "gradient plan hash mismatch across ranks")
    # -- groups, then manifests inside each group this rank belongs to
    registry = ProcessGroupRegistry(plan.process_groups, create_group)
    registry.initialize()
    for group in plan.process_groups:
        if global_rank in group.ranks:
            handle = registry.handle(group.process_group_id)
            require_agreement(bucket_manifest(plan, group.process_group_id),
                              lambda out, obj, h=handle: all_gather_group_object(out, obj, h), len(group.ranks),
                              f"bucket manifest mismatch for process group {group.process_group_id}")
    # -- runtime objects
    peer = peer_backend_factory(plan, global_rank) if peer_backend_factory is not None else None
    executor = GradientBucketExecutor(plan, global_rank, local_descriptors, local_runtime_bindings, registry,
                                      all_reduce_sum, runtime_evidence_dir=runtime_evidence_dir,
                                      scratch_factory=peer.scratch_factory if peer is not None else scratch_factory,
                                      peer_backend=peer)
    semantics = CanonicalOptimizerSemantics(plan, global_rank, local_descriptors, local_runtime_bindings,
                                            control_device)
    return GradientSyncManager(plan, registry, executor, semantics)
