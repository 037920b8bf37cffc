"""Parallel state of one rank in an HPP run: who am I, who are my tensor-/data-parallel peers,
which ranks feed me activations and which consume mine.

The reference keeps this in module-level globals (`mpu`, eth/runtime/megatron/mpu/initialize.py:
group registry :757-786, all TP/DP groups of all pipelines created on every rank :316-410, this
rank's groups / parent-child maps :93-314, cross-check against the canonical topology
:176-230 of grad_sync/topology.py). Here it is one object built from the canonical topology, with
the process-group factory injected (NCCL, Gloo, or a fake in unit tests).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

from .grad_sync.topology import (CanonicalStageTopology, CanonicalTopology, build_canonical_topology,
                                 build_mpu_rank_facts, validate_mpu_rank_facts)


class GroupRegistry:
    """Process groups keyed by their sorted rank tuple; created once, then frozen."""

    def __init__(self, create_group: Callable[[Tuple[int, ...]], object]):
        self._create = create_group
        self._groups: Dict[Tuple[int, ...], object] = {}
        self._frozen = False

    def create_all(self, rank_tuples) -> None:
        if self._frozen:
            raise RuntimeError("group registry is frozen")
        for ranks in sorted(set(tuple(r) for r in rank_tuples)):
            if ranks not in self._groups:
                self._groups[ranks] = self._create(ranks)
        self._frozen = True

    def get(self, ranks: Tuple[int, ...]):
        ranks = tuple(ranks)
        if ranks not in self._groups:
            raise KeyError(f"process group {ranks} was not created at initialisation")
        return self._groups[ranks]

    def __len__(self):
        return len(self._groups)


class ParallelState:
    def __init__(self, normalized_config: dict, rank: int, create_group: Optional[Callable] = None,
                 topology: Optional[CanonicalTopology] = None):
        self.config = normalized_config
        self.rank = rank
        self.world_size = normalized_config["world_size"]
        self.topology = topology or build_canonical_topology(normalized_config)
        self.stage: CanonicalStageTopology = self.topology.stage_for_rank(rank)
        self.coord = self.stage.coordinate(rank)
        self.pipeline_id, self.stage_id = self.stage.pipeline_id, self.stage.stage_id
        self.pipe = normalized_config["pipe"][self.pipeline_id]
        self.num_stages = self.pipe["num_stages"]
        self.tp_size, self.dp_size = self.stage.tp_degree, self.stage.dp_degree
        self.tp_rank, self.dp_rank = self.coord.tp_rank, self.coord.dp_rank
        facts = self.topology.expected_rank_facts(rank)
        self.tp_group_ranks = facts["tp_group_ranks"]
        self.dp_group_ranks = facts["dp_group_ranks"]
        self.registry = GroupRegistry(create_group or (lambda ranks: None))
        # every TP / DP tuple of every stage of every pipeline, in one global order on all ranks
        self.registry.create_all(self.topology.all_group_rank_tuples())
        self.tp_group = self.registry.get(self.tp_group_ranks)
        self.dp_group = self.registry.get(self.dp_group_ranks)
        validate_mpu_rank_facts(self.topology, build_mpu_rank_facts(
            rank, self.pipeline_id, self.stage_id, self.stage.global_op_begin, self.stage.global_op_end,
            self.stage.stage_ranks, self.tp_group_ranks, self.dp_group_ranks, facts["cp_group_ranks"]))

    # -- pipeline neighbours
    @property
    def is_first_stage(self) -> bool:
        return self.stage_id == 0

    @property
    def is_last_stage(self) -> bool:
        return self.stage_id == self.num_stages - 1

    def neighbour(self, delta: int) -> Optional[CanonicalStageTopology]:
        s = self.stage_id + delta
        if not 0 <= s < self.num_stages:
            return None
        return self.topology.stage(self.pipeline_id, s)

    @property
    def op_range(self) -> Tuple[int, int]:
        return self.stage.global_op_begin, self.stage.global_op_end

    @property
    def micro_batch_size(self) -> int:
        return self.pipe["micro_batch_size"]

    @property
    def local_micro_batch(self) -> int:
        return self.pipe["micro_batch_size"] // self.dp_size

    @property
    def num_microbatches(self) -> int:
        return self.pipe["global_batch_size"] // self.pipe["micro_batch_size"]

    @property
    def recompute_ops(self):
        return self.pipe["recompute_ops"][self.stage_id]

    def max_tp_over_all_pipelines(self) -> int:
        return max(s.tp_degree for s in self.topology.stages)
