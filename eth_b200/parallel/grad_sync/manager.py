"""Lifecycle of canonical gradient synchronisation on one rank.

  gather descriptors over the world -> plan fragments -> build the bucket plan -> all ranks compare
  the plan hash -> create every process group in one global order -> per group, compare bucket
  manifests -> build the executor and the optimizer semantics.

Every collective is an injected callable, so the whole lifecycle runs in unit tests with
in-memory fakes and in multi-process CPU tests over Gloo
(reference: eth/runtime/megatron/grad_sync/manager.py:122-214).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path

from .buckets import ProcessGroupRegistry, build_gradient_sync_plan
from .executor import GradientBucketExecutor
from .optimizer_semantics import CanonicalOptimizerSemantics
from .planner import plan_canonical_fragments


def dump_gradient_sync_plan(plan, path) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(asdict(plan), indent=2, sort_keys=True) + "\n", encoding="utf-8")


@dataclass(frozen=True)
class GradientSyncManager:
    plan: object
    registry: ProcessGroupRegistry
    executor: GradientBucketExecutor
    optimizer_semantics: CanonicalOptimizerSemantics

    def execute(self, normalization_scale=1.0):
        self.executor.execute(normalization_scale=normalization_scale)

    def _via_registry(self, broadcast):
        def call(payload, source_rank, process_group_id, _ranks, _tag, _me):
            broadcast(payload, source_rank, self.registry.handle(process_group_id))
        return call

    def synchronize_parameters(self, broadcast):
        self.optimizer_semantics.synchronize_parameters(self._via_registry(broadcast))

    def synchronize_shared_root_gradients(self, broadcast):
        self.optimizer_semantics.synchronize_shared_root_gradients(self._via_registry(broadcast))

    def synchronize_optimizer_state(self, optimizer, broadcast, all_gather_group_object):
        sem = self.optimizer_semantics
        for group in self.plan.process_groups:
            if sem.global_rank not in group.ranks:
                continue
            mine = sem.optimizer_state_manifest_for_group(group.process_group_id, optimizer.state_for_model_parameter)
            got = [None] * len(group.ranks)
            all_gather_group_object(got, mine, self.registry.handle(group.process_group_id))
            if any(x != mine for x in got):
                raise ValueError(f"optimizer state manifest mismatch for process group "
                                 f"{group.process_group_id}: {tuple(got)}")
        sem.synchronize_optimizer_state(optimizer.state_for_model_parameter, self._via_registry(broadcast))


def initialize_gradient_sync(*, local_descriptors, local_runtime_bindings, topology, model_impl, manifest_hash,
                             sync_mode, bucket_cap_bytes, global_rank, all_gather_object,
                             all_gather_group_object, create_group, all_reduce_sum, control_device="cpu",
                             runtime_evidence_dir=None, scratch_factory=None, peer_backend_factory=None):
    gathered = [None] * topology.world_size
    all_gather_object(gathered, tuple(local_descriptors))
    if any(x is None for x in gathered):
        raise ValueError("gradient metadata gather returned an incomplete world")
    everything = tuple(d for per_rank in gathered for d in per_rank)
    pipelines = tuple(sorted({s.pipeline_id for s in topology.stages}))
    fragments = plan_canonical_fragments(everything, expected_pipeline_ids=pipelines)
    plan = build_gradient_sync_plan(fragments, sync_mode, bucket_cap_bytes, model_impl, manifest_hash,
                                    topology.fingerprint)
    hashes = [None] * topology.world_size
    all_gather_object(hashes, plan.global_plan_hash)
    if len(set(hashes)) != 1:
        raise ValueError(f"gradient plan hash mismatch across ranks: {tuple(hashes)}")
    registry = ProcessGroupRegistry(plan.process_groups, create_group)
    registry.initialize()
    for group in plan.process_groups:
        if global_rank not in group.ranks:
            continue
        mine = tuple((b.semantic_hash, b.exact_numel, b.grad_dtype, len(b.placements))
                     for b in plan.global_bucket_order if b.process_group_id == group.process_group_id)
        got = [None] * len(group.ranks)
        all_gather_group_object(got, mine, registry.handle(group.process_group_id))
        if any(x != mine for x in got):
            raise ValueError(f"bucket manifest mismatch for process group {group.process_group_id}: {tuple(got)}")
    peer = peer_backend_factory(plan, global_rank) if peer_backend_factory is not None else None
    executor = GradientBucketExecutor(plan, global_rank, local_descriptors, local_runtime_bindings, registry,
                                      all_reduce_sum, runtime_evidence_dir=runtime_evidence_dir,
                                      scratch_factory=(peer.scratch_factory if peer is not None else scratch_factory),
                                      peer_backend=peer)
    semantics = CanonicalOptimizerSemantics(plan, global_rank, local_descriptors, local_runtime_bindings,
                                            control_device)
    return GradientSyncManager(plan, registry, executor, semantics)
