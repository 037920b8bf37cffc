"""Immutable canonical topology of an HPP config: which ranks form each stage and how they are
arranged into tensor-/data-/context-parallel groups.

Ranks are handed out pipeline by pipeline and stage by stage. Inside a stage a rank is a
mixed-radix number over (dp, cp, tp) with tp the fastest digit (reference:
eth/runtime/megatron/grad_sync/topology.py:93-173, eth/runtime/megatron/mpu/initialize.py:153-197),
so a stage is fully described by its first rank and its three degrees: coordinates, group
membership and the rank at a coordinate are arithmetic on that description (`StageGrid`).
The stage record additionally carries the expanded group lists, because plans and evidence files
quote them.
"""
from __future__ import annotations

from dataclasses import dataclass
from itertools import product
from typing import Dict, Iterator, Tuple

AXES = ("tp", "dp", "cp")


@dataclass(frozen=True)
class RankCoordinate:
    global_rank: int
    tp_rank: int
    dp_rank: int
    cp_rank: int


@dataclass(frozen=True)
class StageGrid:
    """first rank + degrees; rank = first + (dp * CP + cp) * TP + tp."""
    first_rank: int
    tp: int
    dp: int
    cp: int

    @property
    def size(self) -> int:
        return self.tp * self.dp * self.cp

    def rank_at(self, tp: int, dp: int, cp: int = 0) -> int:
        return self.first_rank + (dp * self.cp + cp) * self.tp + tp

    def coordinate_of(self, rank: int) -> RankCoordinate:
        index = rank - self.first_rank
        if not 0 <= index < self.size:
            raise KeyError(rank)
        rest, t = divmod(index, self.tp)
        d, c = divmod(rest, self.cp)
        return RankCoordinate(rank, t, d, c)

    def line(self, axis: str, at: RankCoordinate) -> Tuple[int, ...]:
        """Ranks that differ from `at` only in `axis`: the group of that kind `at` belongs to."""
        fixed = {"tp": at.tp_rank, "dp": at.dp_rank, "cp": at.cp_rank}
        out = []
        for i in range(getattr(self, axis)):
            fixed[axis] = i
            out.append(self.rank_at(fixed["tp"], fixed["dp"], fixed["cp"]))
        return tuple(out)

    def lines(self, axis: str) -> Tuple[Tuple[int, ...], ...]:
        """All groups of one kind, each once, ordered by their first rank's coordinates (dp, cp, tp)."""
        seen, out = set(), []
        for d, c, t in product(range(self.dp), range(self.cp), range(self.tp)):
            group = self.line(axis, RankCoordinate(self.rank_at(t, d, c), t, d, c))
            if group not in seen:
                seen.add(group)
                out.append(group)
        order = {"tp": lambda g: g, "dp": lambda g: self._key_cp_tp(g[0]), "cp": lambda g: self._key_dp_tp(g[0])}
        return tuple(sorted(out, key=order[axis]))

    def _key_cp_tp(self, rank):
        c = self.coordinate_of(rank)
        return (c.cp_rank, c.tp_rank)

    def _key_dp_tp(self, rank):
        c = self.coordinate_of(rank)
        return (c.dp_rank, c.tp_rank)

    def ranks(self) -> Iterator[int]:
        return iter(range(self.first_rank, self.first_rank + self.size))


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

    @property
    def grid(self) -> StageGrid:
        return StageGrid(self.stage_ranks[0], self.tp_degree, self.dp_degree, self.cp_degree)

    def coordinate(self, global_rank: int) -> RankCoordinate:
        try:
            return self.grid.coordinate_of(global_rank)
        except KeyError:
            raise KeyError(f"rank {global_rank} is not in pipeline {self.pipeline_id} stage {self.stage_id}") from None

    def rank_of(self, tp_rank: int, dp_rank: int, cp_rank: int = 0) -> int:
        return self.grid.rank_at(tp_rank, dp_rank, cp_rank)

    @classmethod
    def from_grid(cls, pipeline_id, stage_id, op_begin, op_count, grid: StageGrid) -> "CanonicalStageTopology":
        return cls(pipeline_id=pipeline_id, stage_id=stage_id, global_op_begin=op_begin,
                   global_op_end=op_begin + op_count, stage_ranks=tuple(grid.ranks()), tp_degree=grid.tp,
                   dp_degree=grid.dp, cp_degree=grid.cp,
                   rank_coordinates=tuple(grid.coordinate_of(r) for r in grid.ranks()),
                   tp_group_ranks_by_coordinate=grid.lines("tp"), dp_group_ranks_by_coordinate=grid.lines("dp"),
                   cp_group_ranks_by_coordinate=grid.lines("cp"))


@dataclass(frozen=True)
class CanonicalTopology:
    world_size: int
    stages: Tuple[CanonicalStageTopology, ...]
    fingerprint: str

    def stage(self, pipeline_id: int, stage_id: int) -> CanonicalStageTopology:
        for s in self.stages:
            if (s.pipeline_id, s.stage_id) == (pipeline_id, stage_id):
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
        """Every TP / DP / CP group of every stage, each once, sorted: the creation order."""
        every = {g for s in self.stages for axis in AXES for g in s.grid.lines(axis)}
        return tuple(sorted(every))

    def expected_rank_facts(self, global_rank: int) -> Dict[str, object]:
        """What the process-group runtime must report for `global_rank` (see `validate_mpu_rank_facts`)."""
        s = self.stage_for_rank(global_rank)
        at = s.coordinate(global_rank)
        facts: Dict[str, object] = {"global_rank": global_rank}
        for key in ("pipeline_id", "stage_id", "global_op_begin", "global_op_end", "stage_ranks",
                    "tp_degree", "dp_degree", "cp_degree"):
            facts[key] = getattr(s, key)
        for axis in AXES:
            facts[f"{axis}_rank"] = getattr(at, f"{axis}_rank")
            facts[f"{axis}_group_ranks"] = s.grid.line(axis, at)
        return facts


def build_canonical_topology(normalized_config) -> CanonicalTopology:
    stages, cursor = [], 0
    for pipeline_id, pipe in enumerate(normalized_config["pipe"]):
        first_op = 0
        degree = {axis: pipe[f"{name}_parallel_size_of_each_op"] for axis, name in
                  (("tp", "model"), ("dp", "data"), ("cp", "context"))}
        for stage_id, op_count in enumerate(pipe["num_ops_in_each_stage"]):
            grid = StageGrid(cursor, degree["tp"][stage_id][0], degree["dp"][stage_id][0], degree["cp"][stage_id][0])
            if grid.size != pipe["num_gpus"][stage_id]:
                raise ValueError(f"pipeline {pipeline_id} stage {stage_id} has topology size {grid.size}, "
                                 f"expected {pipe['num_gpus'][stage_id]}")
            stages.append(CanonicalStageTopology.from_grid(pipeline_id, stage_id, first_op, op_count, grid))
            cursor += grid.size
            first_op += op_count
    if cursor != normalized_config["world_size"]:
        raise ValueError(f"canonical topology covers {cursor} ranks, expected world size "
                         f"{normalized_config['world_size']}")
    return CanonicalTopology(world_size=cursor, stages=tuple(stages),
                             fingerprint=normalized_config["topology_fingerprint"])


def build_mpu_rank_facts(global_rank, pipeline_id, stage_id, global_op_begin, global_op_end,
                         stage_ranks, tp_group_ranks, dp_group_ranks, cp_group_ranks):
    """Facts as seen by the process-group runtime, in the same shape as `expected_rank_facts`."""
    lists = {"stage_ranks": tuple(stage_ranks), "tp_group_ranks": tuple(tp_group_ranks),
             "dp_group_ranks": tuple(dp_group_ranks), "cp_group_ranks": tuple(cp_group_ranks)}
    for name, ranks in lists.items():
        if list(ranks) != sorted(ranks):
            raise ValueError(f"rank {global_rank} {name} must be sorted")
        if global_rank not in ranks:
            raise ValueError(f"rank {global_rank} is missing from {name}")
    facts = {"global_rank": global_rank, "pipeline_id": pipeline_id, "stage_id": stage_id,
             "global_op_begin": global_op_begin, "global_op_end": global_op_end, "stage_ranks": lists["stage_ranks"]}
    for axis in AXES:
        group = lists[f"{axis}_group_ranks"]
        facts[f"{axis}_degree"] = len(group)
        facts[f"{axis}_rank"] = group.index(global_rank)
        facts[f"{axis}_group_ranks"] = group
    return facts


def validate_mpu_rank_facts(topology: CanonicalTopology, actual) -> None:
    rank = actual.get("global_rank")
    expected = topology.expected_rank_facts(rank)
    where = f"rank {rank} pipeline {expected['pipeline_id']} stage {expected['stage_id']}"
    wrong = [k for k, v in expected.items() if actual.get(k) != v]
    if wrong:
        k = wrong[0]
        raise ValueError(f"MPU topology mismatch for {where}: {k} expected {expected[k]}, got {actual.get(k)}")
