"""Which stage to fix, which stage to lean on, and which moves to try first.

Reference policy (eth/searching/policy.py:32-228): the target is the stage that uses the most
memory if any stage is over its device limit, otherwise the slowest stage; the partner is the
stage with the most efficiently usable idle time (when time is the problem) or the least memory
(when memory is); moves are ordered by what dominates the target's cost -- ideal compute,
efficiency loss, or recomputation. Visited plans are remembered by key.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Set, Tuple

from .actions import CATALOGUE, Move


@dataclass
class StageView:
    """What the policy looks at for one stage (filled from an `OpStageEval`)."""
    index: int
    time_us: float
    compute_us: float
    recompute_us: float
    memory_mb: float
    limit_mb: float
    gpus: int

    @property
    def over_memory(self) -> bool:
        return self.memory_mb > self.limit_mb


def views_of(evals, plan) -> List[StageView]:
    out = []
    for i, (ev, st) in enumerate(zip(evals, plan.stages)):
        recompute = ev.time_us - ev.compute_us if ev is not None else 0.0
        out.append(StageView(i, ev.time_us, ev.compute_us, max(0.0, recompute), ev.memory_mb, ev.memory_limit_mb, st.gpus))
    return out


def target_stage(views: Sequence[StageView]) -> Tuple[int, str]:
    """(stage index, 'memory' | 'time'): what has to give."""
    over = [v for v in views if v.over_memory]
    if over:
        return max(over, key=lambda v: v.memory_mb / v.limit_mb).index, "memory"
    return max(views, key=lambda v: v.time_us).index, "time"


def partner_stages(views: Sequence[StageView], target: int, problem: str) -> List[int]:
    """Other stages, most promising first. For a time problem: the most idle time per iteration,
    weighted by how much of the stage's time is real compute (idle time next to a stage that is
    itself mostly overhead is worth less). For a memory problem: the most free memory."""
    others = [v for v in views if v.index != target]
    if problem == "memory":
        ranked = sorted(others, key=lambda v: v.memory_mb / v.limit_mb)
    else:
        slowest = max(v.time_us for v in views)
        def usable_idle(v):
            efficiency = v.compute_us / v.time_us if v.time_us > 0 else 0.0
            return (slowest - v.time_us) * efficiency
        ranked = sorted(others, key=lambda v: -usable_idle(v))
    # adjacent partners first among equals: fewer stages have to pass work along
    return [v.index for v in sorted(ranked, key=lambda v: (ranked.index(v), abs(v.index - target)))]


def ordered_moves(view: StageView, problem: str, allow_gpu_moves: bool, allow_exchange: bool) -> List[Move]:
    """Moves that relieve `problem`, ordered by what dominates the target stage's time."""
    wanted = "memory" if problem == "memory" else "time"
    pool = [m for m in CATALOGUE if m.helps(wanted)]
    if not allow_gpu_moves:
        pool = [m for m in pool if m.name != "take-gpus"]
    if not allow_exchange:
        pool = [m for m in pool if m.name not in ("tp-up-dp-down", "dp-up-tp-down")]
    overhead = view.time_us - view.compute_us - view.recompute_us
    if view.recompute_us >= max(overhead, 0.25 * view.compute_us):
        priority = ["migrate-ops", "tp-up-dp-down", "take-gpus", "smaller-micro-batch"]   # free memory first
    elif overhead > 0.25 * view.compute_us:
        priority = ["dp-up-tp-down", "larger-micro-batch", "migrate-ops", "take-gpus"]    # win back efficiency
    else:
        priority = ["migrate-ops", "take-gpus", "dp-up-tp-down", "smaller-micro-batch"]   # plain imbalance
    rank = {name: i for i, name in enumerate(priority)}
    return sorted(pool, key=lambda m: rank.get(m.name, len(rank)))


class Visited:
    """Plans already expanded, by key."""

    def __init__(self):
        self._keys: Set[tuple] = set()

    def add(self, plan) -> bool:
        k = plan.key()
        if k in self._keys:
            return False
        self._keys.add(k)
        return True

    def __len__(self):
        return len(self._keys)
