"""Op-granular description of a pipeline during search.

The reference keeps `SearchStage` / `SearchConfig` objects with per-op TP, DP and algo lists
(eth/searching/state.py:7-53). Here a pipeline is a tuple of immutable `StagePlan`s, each a
half-open range of global op indices with one TP x DP shape and a per-op recompute mask, so plans
hash, compare and copy cheaply (the local search keeps visited sets of them).

Global op indices follow the manifest: 0 = embedding, then 10 ops per layer, then final-layernorm
and gpt-post-process. A cut may fall between any two ops (`op` grain), after a sub-block
(`block` grain: after the attention half or the MLP half of a layer) or between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Iterable, List, Sequence, Tuple

from ..contract.config import LAYER_OPS

OPS_PER_LAYER = len(LAYER_OPS)
ATTENTION_HALF = 5          # ops of a layer up to and including enc-post-attention-dropout
GRAINS = ("op", "block", "layer")


def total_ops(num_layers: int) -> int:
    return 1 + OPS_PER_LAYER * num_layers + 2


def op_position(op_index: int, num_layers: int) -> Tuple[str, int]:
    """('pre', 0) | ('layer', position inside the layer) | ('post', 0 or 1)."""
    if op_index == 0:
        return "pre", 0
    body = OPS_PER_LAYER * num_layers
    if op_index <= body:
        return "layer", (op_index - 1) % OPS_PER_LAYER
    return "post", op_index - body - 1


def legal_cuts(num_layers: int, grain: str) -> List[int]:
    """Global op indices at which a stage may begin (besides 0), in increasing order."""
    if grain not in GRAINS:
        raise ValueError(f"unknown op grain {grain!r}")
    n = total_ops(num_layers)
    if grain == "op":
        return list(range(1, n))
    cuts = []
    for layer in range(num_layers):
        first = 1 + layer * OPS_PER_LAYER
        if layer > 0:
            cuts.append(first)
        if grain == "block":
            cuts.append(first + ATTENTION_HALF)
    return cuts


@dataclass(frozen=True)
class StagePlan:
    op_begin: int
    op_end: int
    gpus: int
    tp: int
    dp: int
    gpu_types: Tuple[str, ...]           # distinct GPU types among the stage's devices
    recompute: Tuple[int, ...] = ()      # 0/1 per op of the stage; () = none
    algo: int = 0                        # 0: usual column-then-row sharding of the TP GEMMs, 1: swapped

    @property
    def num_ops(self) -> int:
        return self.op_end - self.op_begin

    def mask(self) -> Tuple[int, ...]:
        return self.recompute if self.recompute else (0,) * self.num_ops


@dataclass(frozen=True)
class PipelinePlan:
    stages: Tuple[StagePlan, ...]
    mbs: int

    @property
    def num_gpus(self) -> int:
        return sum(s.gpus for s in self.stages)

    def with_stage(self, index: int, stage: StagePlan) -> "PipelinePlan":
        stages = list(self.stages)
        stages[index] = stage
        return PipelinePlan(tuple(stages), self.mbs)

    def moved_boundary(self, left: int, new_cut: int) -> "PipelinePlan":
        """The boundary between stage `left` and `left + 1` moved to op index `new_cut`."""
        a, b = self.stages[left], self.stages[left + 1]
        if not a.op_begin < new_cut < b.op_end:
            raise ValueError("a boundary move may not empty a stage")
        stages = list(self.stages)
        stages[left] = replace(a, op_end=new_cut, recompute=())
        stages[left + 1] = replace(b, op_begin=new_cut, recompute=())
        return PipelinePlan(tuple(stages), self.mbs)

    def key(self) -> tuple:
        return (self.mbs,) + tuple((s.op_begin, s.op_end, s.tp, s.dp, s.gpus, s.algo) for s in self.stages)


def plan_from_layers(layers: Sequence[int], shapes: Iterable[Tuple[int, int, int, Tuple[str, ...]]], mbs: int,
                     num_layers: int) -> PipelinePlan:
    """Layer-granular plan (what the boundary DP produces): stage i holds `layers[i]` whole layers,
    the first stage also the embedding, the last one the two tail ops."""
    stages, cursor = [], 0
    shapes = list(shapes)
    for i, (count, (gpus, tp, dp, types)) in enumerate(zip(layers, shapes)):
        end = cursor + count * OPS_PER_LAYER + (1 if i == 0 else 0) + (2 if i == len(shapes) - 1 else 0)
        stages.append(StagePlan(cursor, end, gpus, tp, dp, tuple(types)))
        cursor = end
    if cursor != total_ops(num_layers):
        raise ValueError("layer counts do not cover the model")
    return PipelinePlan(tuple(stages), mbs)
