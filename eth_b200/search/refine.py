"""Multi-hop local search over op-granular pipeline plans.

Starting from an initial plan (the layer-granular optimum of the boundary DP, or a balanced
split, or a plan read from JSON), repeatedly: find the stage that has to give (policy), order the
moves that relieve it, generate neighbours, and take the first neighbour that is feasible and
better. When no single move improves, recurse into the best few neighbours up to `max_hops` deep,
so that a move that is bad on its own (e.g. a smaller micro-batch) can be followed by the move it
enables. Bounded by a deadline. (reference: multi_hop_search / trial, eth/searching/search.py:170-261,
374-446.)
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

from .actions import change_micro_batch, exchange_tp_dp, migrate_ops, move_gpus, swap_sharding
from .cost_model import CostModel
from .policy import Visited, ordered_moves, partner_stages, target_stage, views_of
from .state import PipelinePlan


@dataclass
class ScoredPlan:
    plan: PipelinePlan
    evals: list
    feasible: bool

    @property
    def stage_times(self) -> List[float]:
        return [e.time_us for e in self.evals]

    def per_sample_us(self) -> float:
        """Steady-state time per sample, with fill/drain as a small tie-breaker."""
        if not self.feasible:
            return float("inf")
        t = self.stage_times
        return max(t) / self.plan.mbs + 1e-6 * sum(t) / self.plan.mbs


class Refiner:
    def __init__(self, cost: CostModel, num_layers: int, grain: str, mbs_candidates: Sequence[int], max_tp: int,
                 heads: int, hidden: int, max_hops: int = 7, allow_gpu_moves: bool = False,
                 allow_exchange: bool = True, branch: int = 3):
        self.cost, self.L, self.grain = cost, num_layers, grain
        self.mbs_candidates, self.max_tp, self.heads, self.hidden = list(mbs_candidates), max_tp, heads, hidden
        self.max_hops, self.allow_gpu_moves, self.allow_exchange, self.branch = max_hops, allow_gpu_moves, allow_exchange, branch
        self.evaluated = 0
        self.trace: List[Tuple[float, str, float]] = []     # (seconds, move, per-sample us) of every improvement

    # ------------------------------------------------------------------ evaluation
    def score(self, plan: PipelinePlan) -> ScoredPlan:
        n = len(plan.stages)
        evals, ok = [], True
        for i, st in enumerate(plan.stages):
            nxt = plan.stages[i + 1] if i + 1 < n else None
            ev = self.cost.stage_eval_ops(st, plan.mbs, n - 1 - i, nxt)
            if ev is None:
                ok = False
                break
            evals.append(ev)
        self.evaluated += 1
        return ScoredPlan(plan, evals, ok)

    def with_recompute(self, scored: ScoredPlan) -> PipelinePlan:
        """The plan with the recompute masks the cost model settled on."""
        from dataclasses import replace
        stages = tuple(replace(st, recompute=ev.recompute if any(ev.recompute) else ())
                       for st, ev in zip(scored.plan.stages, scored.evals))
        return PipelinePlan(stages, scored.plan.mbs)

    # ------------------------------------------------------------------ neighbourhood
    def neighbours(self, scored: ScoredPlan):
        """(move name, plan) in the order the policy wants them tried."""
        plan = scored.plan
        views = views_of(scored.evals, plan)
        target, problem = target_stage(views)
        partners = partner_stages(views, target, problem)
        for move in ordered_moves(views[target], problem, self.allow_gpu_moves, self.allow_exchange):
            if move.name == "migrate-ops":
                for partner in partners:
                    for p in migrate_ops(plan, target, partner, self.L, self.grain):
                        yield move.name, p
            elif move.name in ("tp-up-dp-down", "dp-up-tp-down"):
                want_tp_up = move.name == "tp-up-dp-down"
                for p in exchange_tp_dp(plan, target, self.max_tp, self.heads, self.hidden):
                    if (p.stages[target].tp > plan.stages[target].tp) == want_tp_up:
                        yield move.name, p
            elif move.name == "swap-sharding":
                for p in swap_sharding(plan, target):
                    yield move.name, p
            elif move.name == "take-gpus":
                for partner in partners:
                    for p in move_gpus(plan, partner, target, self.max_tp, self.heads, self.hidden):
                        yield move.name, p
            else:
                smaller = move.name == "smaller-micro-batch"
                for p in change_micro_batch(plan, self.mbs_candidates, self.max_tp, self.heads, self.hidden):
                    if (p.mbs < plan.mbs) == smaller:
                        yield move.name, p

    # ------------------------------------------------------------------ search
    def refine(self, start: PipelinePlan, deadline: float) -> ScoredPlan:
        t0 = time.time()
        best = self.score(start)
        visited = Visited()
        visited.add(start)
        improved = True
        while improved and time.time() < deadline:
            improved = False
            found = self._hop(best, best.per_sample_us(), self.max_hops, visited, deadline, [])
            if found is not None:
                best, path = found
                self.trace.append((time.time() - t0, " > ".join(path), best.per_sample_us()))
                improved = True
        return best

    def _hop(self, node: ScoredPlan, bar: float, hops_left: int, visited: Visited, deadline: float, path):
        """First plan within `hops_left` moves of `node` that beats `bar`, or None."""
        if hops_left <= 0 or not node.evals:
            return None
        fringe = []
        for name, plan in self.neighbours(node):
            if time.time() > deadline:
                return None
            if not visited.add(plan):
                continue
            sp = self.score(plan)
            if sp.feasible and sp.per_sample_us() < bar * (1 - 1e-9):
                return sp, path + [name]
            if sp.evals and len(sp.evals) == len(plan.stages):
                fringe.append((sp.per_sample_us() if sp.feasible else float("inf"), len(fringe), name, sp))
        fringe.sort(key=lambda x: x[:2])
        for _, _, name, sp in fringe[: self.branch]:
            if not sp.feasible:
                continue
            hit = self._hop(sp, bar, hops_left - 1, visited, deadline, path + [name])
            if hit is not None:
                return hit
        return None
