"""Moves of the local search over pipeline plans.

The reference explores configurations with a set of primitives, each tagged with the resources it
is expected to trade (eth/searching/actions.py:41-53, 1467-1496): migrating ops out of a
bottleneck stage toward a partner stage, hop by hop, at op / block / layer granularity (:164-320),
changing the micro-batch size and re-picking TP x DP (:1138-1222), exchanging TP against DP inside
a stage (:1435-1462) and moving GPUs between stages (:919-1118). The same moves exist here as pure
functions `PipelinePlan -> [PipelinePlan]`; evaluation and choice are left to `refine.py`.

Effect signature of a move, per resource, as seen from the stage it is applied to:
'+' the move is expected to increase it, '-' to decrease it, '0' to leave it alone.
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass, replace
from typing import Callable, Dict, Iterator, List, Sequence, Tuple

from .state import PipelinePlan, StagePlan, legal_cuts

RESOURCES = ("time", "memory", "devices", "workload", "efficiency", "comm")


@dataclass(frozen=True)
class Move:
    name: str
    effect: Dict[str, str]                       # resource -> '+', '-' or '0' for the target stage
    generate: Callable[..., Iterator[PipelinePlan]]

    def helps(self, resource: str) -> bool:
        return self.effect.get(resource) == "-"


def _effects(**kw) -> Dict[str, str]:
    out = {r: "0" for r in RESOURCES}
    out.update(kw)
    return out


# ------------------------------------------------------------------------------------------
# migrate ops from a stage toward a partner, one boundary at a time
# ------------------------------------------------------------------------------------------
def _shifted_cut(cuts: Sequence[int], current: int, direction: int, lo: int, hi: int):
    """Next legal cut position after `current` in `direction` that keeps both neighbours non-empty."""
    i = bisect.bisect_left(cuts, current)
    j = i + direction if (i < len(cuts) and cuts[i] == current) else (i if direction > 0 else i - 1)
    if 0 <= j < len(cuts) and lo < cuts[j] < hi:
        return cuts[j]
    return None


def migrate_ops(plan: PipelinePlan, source: int, partner: int, num_layers: int, grain: str,
                max_steps: int = 4) -> Iterator[PipelinePlan]:
    """Shrink stage `source` by moving its boundary toward `partner`: 1, 2, ... grain units leave
    `source`; every stage between the two passes the same amount on, so only `source` loses work
    and only `partner` gains it (the reference's hop-by-hop migration)."""
    if source == partner:
        return
    cuts = legal_cuts(num_layers, grain)
    step = 1 if partner > source else -1
    current = plan
    for _ in range(max_steps):
        moved = current
        ok = True
        s = source
        while s != partner:
            # boundary between s and s + step, moved so that stage s gives one unit to s + step
            left = min(s, s + step)
            a, b = moved.stages[left], moved.stages[left + 1]
            new_cut = _shifted_cut(cuts, a.op_end, -step, a.op_begin, b.op_end)
            if new_cut is None:
                ok = False
                break
            moved = moved.moved_boundary(left, new_cut)
            s += step
        if not ok:
            return
        current = moved
        yield current


# ------------------------------------------------------------------------------------------
# shape of a stage: TP x DP exchange, and GPUs moving between stages
# ------------------------------------------------------------------------------------------
def exchange_tp_dp(plan: PipelinePlan, index: int, max_tp: int, heads: int, hidden: int) -> Iterator[PipelinePlan]:
    """Same GPUs, TP doubled and DP halved or the other way round."""
    st = plan.stages[index]
    for tp, dp in ((st.tp * 2, st.dp // 2), (st.tp // 2, st.dp * 2)):
        if tp >= 1 and dp >= 1 and tp * dp == st.gpus and tp <= max_tp and heads % tp == 0 and hidden % tp == 0 \
                and plan.mbs % dp == 0 and tp in (1, 2, 4, 8):
            yield plan.with_stage(index, replace(st, tp=tp, dp=dp, recompute=()))


def move_gpus(plan: PipelinePlan, donor: int, receiver: int, max_tp: int, heads: int, hidden: int) -> Iterator[PipelinePlan]:
    """Half of `donor`'s GPUs go to `receiver` (stage sizes stay powers of two only if they were
    equal; otherwise the move is skipped). Types must match: devices keep their identity."""
    a, b = plan.stages[donor], plan.stages[receiver]
    if a.gpus < 2 or a.gpus // 2 != b.gpus or a.gpu_types != b.gpu_types or abs(donor - receiver) != 1:
        return
    give = a.gpus // 2
    for tp_a, dp_a in _shapes(a.gpus - give, max_tp, heads, hidden, plan.mbs):
        for tp_b, dp_b in _shapes(b.gpus + give, max_tp, heads, hidden, plan.mbs):
            stages = list(plan.stages)
            stages[donor] = replace(a, gpus=a.gpus - give, tp=tp_a, dp=dp_a, recompute=())
            stages[receiver] = replace(b, gpus=b.gpus + give, tp=tp_b, dp=dp_b, recompute=())
            yield PipelinePlan(tuple(stages), plan.mbs)


def swap_sharding(plan: PipelinePlan, index: int) -> Iterator[PipelinePlan]:
    """The stage's four tensor-parallel GEMMs in their other sharding (algo 0 <-> 1): qkv / MLP-GEMM-1
    row- instead of column-parallel, dense / MLP-GEMM-2 the other way round. Only the profile says
    which is faster for a given shape (reference: per-op algo fine-tuning, actions.py:1236-1433; one
    value per stage here, as the config contract demands)."""
    st = plan.stages[index]
    if st.tp > 1:
        yield plan.with_stage(index, replace(st, algo=1 - st.algo, recompute=()))


def _shapes(gpus: int, max_tp: int, heads: int, hidden: int, mbs: int) -> List[Tuple[int, int]]:
    return [(tp, gpus // tp) for tp in (1, 2, 4, 8)
            if tp <= max_tp and gpus % tp == 0 and heads % tp == 0 and hidden % tp == 0 and mbs % (gpus // tp) == 0]


def change_micro_batch(plan: PipelinePlan, candidates: Sequence[int], max_tp: int, heads: int, hidden: int) -> Iterator[PipelinePlan]:
    """Neighbouring micro-batch sizes; a stage whose DP no longer divides the new size falls back
    to the widest TP that does (the reference re-picks (tp, dp) per stage after an mbs change)."""
    order = sorted(candidates)
    if plan.mbs not in order:
        return
    i = order.index(plan.mbs)
    for j in (i - 1, i + 1):
        if not 0 <= j < len(order):
            continue
        mbs = order[j]
        stages = []
        for st in plan.stages:
            if mbs % st.dp == 0:
                stages.append(replace(st, recompute=()))
                continue
            fits = _shapes(st.gpus, max_tp, heads, hidden, mbs)
            if not fits:
                stages = None
                break
            tp, dp = max(fits)
            stages.append(replace(st, tp=tp, dp=dp, recompute=()))
        if stages is not None:
            yield PipelinePlan(tuple(stages), mbs)


# The catalogue: what each move trades on the stage it targets (the bottleneck).
CATALOGUE: Tuple[Move, ...] = (
    Move("migrate-ops", _effects(time="-", memory="-", workload="-", comm="0"), migrate_ops),
    Move("tp-up-dp-down", _effects(time="+", memory="-", efficiency="-", comm="+"), exchange_tp_dp),
    Move("dp-up-tp-down", _effects(time="-", memory="+", efficiency="+", comm="-"), exchange_tp_dp),
    Move("take-gpus", _effects(time="-", memory="-", devices="+"), move_gpus),
    Move("smaller-micro-batch", _effects(time="-", memory="-", efficiency="-"), change_micro_batch),
    Move("larger-micro-batch", _effects(time="+", memory="+", efficiency="+"), change_micro_batch),
    Move("swap-sharding", _effects(time="-", memory="-", comm="-"), swap_sharding),
)
