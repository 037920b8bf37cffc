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


def split_stage_ops(n_ops: int, chunks: int, lead: int, tail: int, ops_per_layer: int):
    """Op counts of the `chunks` model chunks of one physical stage. `lead` / `tail` ops (embedding,
    final LayerNorm + head) stay with the first / last chunk; the rest is split into whole layers
    when there are enough of them, else op by op."""
    body = n_ops - lead - tail
    unit = ops_per_layer if body % ops_per_layer == 0 and body // ops_per_layer >= chunks else 1
    units = body // unit
    if units < chunks:
        raise ValueError(f"a stage of {n_ops} ops cannot be cut into {chunks} model chunks")
    base, extra = divmod(units, chunks)
    parts = [(base + (1 if c >= chunks - extra else 0)) * unit for c in range(chunks)]
    parts[0] += lead
    parts[-1] += tail
    return parts


def virtual_stage_ranges(stage_op_counts, chunks: int, ops_per_layer: int):
    """[stage][chunk] -> (op_begin, op_end) for interleaved pipelining: virtual stage c * S + s is
    chunk c of physical stage s, and virtual stages follow each other in the model (reference:
    eth/runtime/megatron/mpu/initialize.py:134-151, 664-674)."""
    stages = len(stage_op_counts)
    parts = [split_stage_ops(n, chunks, 1 if s == 0 else 0, 2 if s == stages - 1 else 0, ops_per_layer)
             for s, n in enumerate(stage_op_counts)]
    # the embedding sits on chunk 0 of stage 0 (the first virtual stage), the tail ops on the last
    # chunk of the last stage (the last virtual stage)
    ranges = [[None] * chunks for _ in range(stages)]
    cursor = 0
    for c in range(chunks):
        for s in range(stages):
            ranges[s][c] = (cursor, cursor + parts[s][c])
            cursor += parts[s][c]
    return ranges


class ParallelState:
    def __init__(self, normalized_config: dict, rank: int, create_group: Optional[Callable] = None,
                 topology: Optional[CanonicalTopology] = None, interleave: int = 1):
        self.config = normalized_config
        self.interleave = max(1, int(interleave))
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

    # -- interleaved pipelining: this rank's model chunks and their neighbours
    @property
    def chunk_ranges(self):
        """Op ranges of this rank's model chunks (one range without interleaving)."""
        if self.interleave == 1:
            return [self.op_range]
        per_layer = self.config["manifest"]["ops_per_layer"]
        return virtual_stage_ranges(self.pipe["num_ops_in_each_stage"], self.interleave, per_layer)[self.stage_id]

    def chunk_neighbour(self, chunk: int, delta: int) -> Optional[CanonicalStageTopology]:
        """Stage that holds the virtual stage before (delta -1) / after (+1) this rank's `chunk`:
        the adjacent physical stage, wrapping from the last stage to the first between chunks."""
        if self.interleave == 1:
            return self.neighbour(delta)
        virtual = chunk * self.num_stages + self.stage_id + delta
        if not 0 <= virtual < self.interleave * self.num_stages:
            return None
        return self.topology.stage(self.pipeline_id, virtual % self.num_stages)

    def is_first_virtual(self, chunk: int) -> bool:
        return self.stage_id == 0 and chunk == 0

    def is_last_virtual(self, chunk: int) -> bool:
        return self.stage_id == self.num_stages - 1 and chunk == self.interleave - 1

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
