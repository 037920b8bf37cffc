"""Immutable canonical topology of an HPP config: which ranks form each stage and how they are
arranged into tensor-/data-/context-parallel groups.

Ranks are laid out pipeline-major, then stage-major; inside a stage the TP index runs fastest,
then CP, then DP (reference: eth/runtime/megatron/grad_sync/topology.py:93-173,
eth/runtime/megatron/mpu/initialize.py:153-197).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple


@dataclass(frozen=True)
class RankCoordinate:
    global_rank: int
    tp_rank: int
    dp_rank: int
    cp_rank: int


@dataclass(frozen=True)
class CanonicalStageTopology:
    pipeline_id: int
    stage_id: int
    global_op_begin: int
    global_op_end: int
    stage_ranks: Tuple[int, ...]
    tp_degree: int
    dp_degree: int
    cp_degree: int
    rank_coordinates: Tuple[RankCoordinate, ...]
    tp_group_ranks_by_coordinate: Tuple[Tuple[int, ...], ...]
    dp_group_ranks_by_coordinate: Tuple[Tuple[int, ...], ...]
    cp_group_ranks_by_coordinate: Tuple[Tuple[int, ...], ...]

    def coordinate(self, global_rank: int) -> RankCoordinate:
        first = self.stage_ranks[0]
        idx = global_rank - first
        if not 0 <= idx < len(self.stage_ranks):
            raise KeyError(f"rank {global_rank} is not in pipeline {self.pipeline_id} stage {self.stage_id}")
        return self.rank_coordinates[idx]

    def rank_of(self, tp_rank: int, dp_rank: int, cp_rank: int = 0) -> int:
        return self.stage_ranks[0] + (dp_rank * self.cp_degree + cp_rank) * self.tp_degree + tp_rank


@dataclass(frozen=True)
class CanonicalTopology:
    world_size: int
    stages: Tuple[CanonicalStageTopology, ...]
    fingerprint: str

    def stage(self, pipeline_id: int, stage_id: int) -> CanonicalStageTopology:
        for s in self.stages:
            if s.pipeline_id == pipeline_id and s.stage_id == stage_id:
                return s
        raise KeyError(f"unknown pipeline {pipeline_id} stage {stage_id}")

    def stage_for_rank(self, global_rank: int) -> CanonicalStageTopology:
        for s in self.stages:
            if s.stage_ranks[0] <= global_rank <= s.stage_ranks[-1]:
                return s
        raise KeyError(f"rank {global_rank} is not present in canonical topology")

    def pipeline_stages(self, pipeline_id: int) -> Tuple[CanonicalStageTopology, ...]:
        return tuple(s for s in self.stages if s.pipeline_id == pipeline_id)

    @property
    def pipeline_ids(self) -> Tuple[int, ...]:
        return tuple(sorted({s.pipeline_id for s in self.stages}))

    def all_group_rank_tuples(self) -> Tuple[Tuple[int, ...], ...]:
        groups = set()
        for s in self.stages:
            groups.update(s.tp_group_ranks_by_coordinate)
            groups.update(s.dp_group_ranks_by_coordinate)
            groups.update(s.cp_group_ranks_by_coordinate)
        return tuple(sorted(groups))

    def expected_rank_facts(self, global_rank: int) -> Dict[str, object]:
        s = self.stage_for_rank(global_rank)
        c = s.coordinate(global_rank)
        pick = lambda groups: next(g for g in groups if global_rank in g)  # noqa: E731
        return {
            "global_rank": global_rank,
            "pipeline_id": s.pipeline_id,
            "stage_id": s.stage_id,
            "global_op_begin": s.global_op_begin,
            "global_op_end": s.global_op_end,
            "stage_ranks": s.stage_ranks,
            "tp_degree": s.tp_degree,
            "dp_degree": s.dp_degree,
            "cp_degree": s.cp_degree,
            "tp_rank": c.tp_rank,
            "dp_rank": c.dp_rank,
            "cp_rank": c.cp_rank,
            "tp_group_ranks": pick(s.tp_group_ranks_by_coordinate),
            "dp_group_ranks": pick(s.dp_group_ranks_by_coordinate),
            "cp_group_ranks": pick(s.cp_group_ranks_by_coordinate),
        }


def _build_stage(pipeline_id, stage_id, op_begin, op_count, first_rank, tp, dp, cp):
    def rank(t, d, c):
        return first_rank + (d * cp + c) * tp + t

    coords = tuple(RankCoordinate(rank(t, d, c), t, d, c)
                   for d in range(dp) for c in range(cp) for t in range(tp))
    tp_groups = tuple(tuple(rank(t, d, c) for t in range(tp)) for d in range(dp) for c in range(cp))
    dp_groups = tuple(tuple(rank(t, d, c) for d in range(dp)) for c in range(cp) for t in range(tp))
    cp_groups = tuple(tuple(rank(t, d, c) for c in range(cp)) for d in range(dp) for t in range(tp))
    size = tp * dp * cp
    return CanonicalStageTopology(
        pipeline_id=pipeline_id, stage_id=stage_id, global_op_begin=op_begin,
        global_op_end=op_begin + op_count, stage_ranks=tuple(range(first_rank, first_rank + size)),
        tp_degree=tp, dp_degree=dp, cp_degree=cp, rank_coordinates=coords,
        tp_group_ranks_by_coordinate=tp_groups, dp_group_ranks_by_coordinate=dp_groups,
        cp_group_ranks_by_coordinate=cp_groups)


def build_canonical_topology(normalized_config) -> CanonicalTopology:
    stages = []
    next_rank = 0
    for pid, pipe in enumerate(normalized_config["pipe"]):
        op_begin = 0
        for sid, n_ops in enumerate(pipe["num_ops_in_each_stage"]):
            tp = pipe["model_parallel_size_of_each_op"][sid][0]
            dp = pipe["data_parallel_size_of_each_op"][sid][0]
            cp = pipe["context_parallel_size_of_each_op"][sid][0]
            if tp * dp * cp != pipe["num_gpus"][sid]:
                raise ValueError(
                    f"pipeline {pid} stage {sid} has topology size {tp * dp * cp}, expected {pipe['num_gpus'][sid]}")
            stages.append(_build_stage(pid, sid, op_begin, n_ops, next_rank, tp, dp, cp))
            next_rank += tp * dp * cp
            op_begin += n_ops
    if next_rank != normalized_config["world_size"]:
        raise ValueError(
            f"canonical topology covers {next_rank} ranks, expected world size {normalized_config['world_size']}")
    return CanonicalTopology(world_size=next_rank, stages=tuple(stages),
                             fingerprint=normalized_config["topology_fingerprint"])


def build_mpu_rank_facts(global_rank, pipeline_id, stage_id, global_op_begin, global_op_end,
                         stage_ranks, tp_group_ranks, dp_group_ranks, cp_group_ranks):
    """Facts as seen by the process-group runtime, in the same shape as `expected_rank_facts`."""
    groups = {"stage_ranks": tuple(stage_ranks), "tp_group_ranks": tuple(tp_group_ranks),
              "dp_group_ranks": tuple(dp_group_ranks), "cp_group_ranks": tuple(cp_group_ranks)}
    for name, ranks in groups.items():
        if ranks != tuple(sorted(ranks)):
            raise ValueError(f"rank {global_rank} {name} must be sorted")
        if global_rank not in ranks:
            raise ValueError(f"rank {global_rank} is missing from {name}")
    return {
        "global_rank": global_rank, "pipeline_id": pipeline_id, "stage_id": stage_id,
        "global_op_begin": global_op_begin, "global_op_end": global_op_end,
        "stage_ranks": groups["stage_ranks"],
        "tp_degree": len(groups["tp_group_ranks"]), "dp_degree": len(groups["dp_group_ranks"]),
        "cp_degree": len(groups["cp_group_ranks"]),
        "tp_rank": groups["tp_group_ranks"].index(global_rank),
        "dp_rank": groups["dp_group_ranks"].index(global_rank),
        "cp_rank": groups["cp_group_ranks"].index(global_rank),
        "tp_group_ranks": groups["tp_group_ranks"], "dp_group_ranks": groups["dp_group_ranks"],
        "cp_group_ranks": groups["cp_group_ranks"],
    }


def validate_mpu_rank_facts(topology: CanonicalTopology, actual) -> None:
    rank = actual.get("global_rank")
    want = topology.expected_rank_facts(rank)
    where = f"rank {rank} pipeline {want['pipeline_id']} stage {want['stage_id']}"
    for key, value in want.items():
        if actual.get(key) != value:
            raise ValueError(f"MPU topology mismatch for {where}: {key} expected {value}, got {actual.get(key)}")
