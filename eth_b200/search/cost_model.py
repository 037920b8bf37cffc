"""Cost model of an HPP configuration on profiled hardware.

Time (reference: eth/searching/cost_model.py:192-217 stage compute, :145-188 boundary P2P,
:799-830 pipeline time): a stage's per-micro-batch time is the sum of its ops' profiled forward +
backward time at the stage's (local micro-batch, TP) -- the maximum over GPU types when a stage
mixes them --, plus one extra forward for recomputed ops, plus the boundary transfer. A pipeline
with n micro-batches costs `max_i (t_i * (n - 1)) + sum_j t_j`; the iteration is the slowest
pipeline.

Two terms the reference leaves out (its `tp_comm` is computed but never added, :220-224, :762)
are modelled here because they matter on NVLink-connected B200s: tensor-parallel reductions that
are not already inside the profiled op time, and the exposed block-wise gradient all-reduce.

Memory (reference :594-625): weights + gradients + fp32 master + two Adam moments, activations
times the number of micro-batches in flight (stages behind + 1), the peak transient of the
largest op, and allocator reserve; recomputed ops keep only their input.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..contract.config import LAYER_OPS
from .profile_db import ProfileDB

PRE_OPS = 1          # encoder-embedding
POST_OPS = 2         # final-layernorm, gpt-post-process
OPS_PER_LAYER = len(LAYER_OPS)


@dataclass(frozen=True)
class StageChoice:
    gpus: int
    tp: int
    dp: int
    gpu_type: str = "default"
    gpu_types: Tuple[str, ...] = ()      # all distinct types of a mixed stage; () = just `gpu_type`
    algo: int = 0                        # sharding choice of the stage's tensor-parallel GEMMs

    def types(self) -> Tuple[str, ...]:
        return self.gpu_types or (self.gpu_type,)


@dataclass
class StageEval:
    time_us: float
    fwd_us: float
    bwd_us: float
    memory_mb: float
    recompute_layers: int
    weights_mb: float


@dataclass
class OpStageEval:
    time_us: float
    fwd_us: float
    bwd_us: float
    memory_mb: float
    recompute: Tuple[int, ...]
    weights_mb: float
    memory_limit_mb: float
    boundary_mb: float

    @property
    def compute_us(self) -> float:
        return self.fwd_us + self.bwd_us


@dataclass
class CostOptions:
    bytes_per_param: float = 2.0          # 16-bit model weights
    grad_bytes_per_param: float = 4.0     # main_grad (fp32 for bf16 runs)
    optimizer_bytes_per_param: float = 12.0  # fp32 master + exp_avg + exp_avg_sq
    memory_reserve_fraction: float = 0.08
    tp_comm_in_op_time: bool = True       # op profiles at TP>1 were taken with the real (fused) reductions
    include_grad_sync: bool = True
    grad_sync_overlap: float = 0.0        # fraction of the gradient all-reduce hidden behind backward
    comm_revised: bool = True             # boundary transfer charged max(prev out, this in) (:748-757)


class CostModel:
    """Evaluates stages, pipelines and whole HPP plans from per-GPU-type profile tables."""

    def __init__(self, profiles: Dict[str, ProfileDB], num_layers: int, device_memory_mb: Dict[str, float],
                 options: Optional[CostOptions] = None):
        self.profiles = profiles
        self.num_layers = num_layers
        self.device_memory_mb = device_memory_mb
        self.opt = options or CostOptions()
        self._layer_cache: Dict[tuple, dict] = {}

    # ------------------------------------------------------------------ per-group aggregates
    def op_rows(self, gpu_types, mbs: int, tp: int, algo: int = 0):
        """The one-layer op table for a stage whose GPUs are of `gpu_types`: per op the slowest
        type's times (the stage advances at the pace of its slowest device, reference
        cost_model.py:192-217); sizes do not depend on the type. None if some type lacks the profile."""
        types = (gpu_types,) if isinstance(gpu_types, str) else tuple(gpu_types)
        key = ("rows", types, mbs, tp, algo)
        if key in self._layer_cache:
            return self._layer_cache[key]
        tables = []
        for t in types:
            db = self.profiles[t]
            if not db.has(mbs, tp, algo):
                self._layer_cache[key] = None
                return None
            tables.append(db.records(mbs, tp, algo))
        rows = tables[0]
        if len(tables) > 1:
            from dataclasses import replace as _replace
            rows = [_replace(r, fwd_us=max(t[i].fwd_us for t in tables), bwd_us=max(t[i].bwd_us for t in tables))
                    for i, r in enumerate(rows)]
        self._layer_cache[key] = rows
        return rows

    def memory_limit_mb(self, gpu_types) -> float:
        types = (gpu_types,) if isinstance(gpu_types, str) else tuple(gpu_types)
        return min(self.device_memory_mb[t] for t in types) * (1.0 - self.opt.memory_reserve_fraction)

    def _groups(self, gpu_type, mbs: int, tp: int, algo: int = 0) -> Optional[dict]:
        """Sums over the three op groups of the one-layer profile: pre (embedding), layer, post.
        `gpu_type` may be one type or a tuple of types (mixed stage)."""
        key = (gpu_type, mbs, tp, algo)
        hit = self._layer_cache.get(key)
        if hit is not None or key in self._layer_cache:
            return hit
        rows = self.op_rows(gpu_type, mbs, tp, algo)
        if rows is None:
            self._layer_cache[key] = None
            return None
        if len(rows) != PRE_OPS + OPS_PER_LAYER + POST_OPS:
            raise ValueError(f"profile for mbs{mbs} tp{tp} has {len(rows)} ops, expected "
                             f"{PRE_OPS + OPS_PER_LAYER + POST_OPS}")
        parts = {"pre": rows[:PRE_OPS], "layer": rows[PRE_OPS:PRE_OPS + OPS_PER_LAYER], "post": rows[-POST_OPS:]}
        out = {}
        for name, rs in parts.items():
            out[name] = {
                "fwd": sum(r.fwd_us for r in rs), "bwd": sum(r.bwd_us for r in rs),
                "weights": sum(r.weights_mb for r in rs), "act": sum(r.activations_mb for r in rs),
                "peak": max(max(r.fwd_reserved_mb, r.bwd_reserved_mb) for r in rs),
                "in": rs[0].input_mb, "out": rs[-1].output_mb,
            }
        self._layer_cache[key] = out
        return out

    # ------------------------------------------------------------------ stage
    def stage_eval(self, choice: StageChoice, mbs: int, first_layer: int, num_layers: int, has_pre: bool,
                   has_post: bool, stages_behind: int, next_choice: Optional[StageChoice] = None,
                   inter_node: bool = False) -> Optional[StageEval]:
        """Cost of a stage holding `num_layers` whole layers (+ embedding / head). None = infeasible
        (no profile for this local micro-batch / TP, or it cannot fit even with full recompute)."""
        if mbs % choice.dp:
            return None
        local = mbs // choice.dp
        g = self._groups(choice.types() if len(choice.types()) > 1 else choice.gpu_type, local, choice.tp)
        if g is None:
            return None
        fwd = num_layers * g["layer"]["fwd"] + (g["pre"]["fwd"] if has_pre else 0) + (g["post"]["fwd"] if has_post else 0)
        bwd = num_layers * g["layer"]["bwd"] + (g["pre"]["bwd"] if has_pre else 0) + (g["post"]["bwd"] if has_post else 0)
        weights = (num_layers * g["layer"]["weights"] + (g["pre"]["weights"] if has_pre else 0)
                   + (g["post"]["weights"] if has_post else 0))
        o = self.opt
        state_mb = weights / o.bytes_per_param * (o.bytes_per_param + o.grad_bytes_per_param + o.optimizer_bytes_per_param)
        inflight = stages_behind + 1
        act_layer = g["layer"]["act"]
        act_fixed = (g["pre"]["act"] if has_pre else 0) + (g["post"]["act"] if has_post else 0)
        peak = max(g["layer"]["peak"], g["post"]["peak"] if has_post else 0, g["pre"]["peak"] if has_pre else 0)
        limit = self.memory_limit_mb(choice.types())
        layer_in = g["layer"]["in"]

        def mem(recomputed: int) -> float:
            kept = (num_layers - recomputed) * act_layer + recomputed * layer_in + act_fixed
            transient = act_layer if recomputed else 0.0
            return state_mb + kept * inflight + transient + peak

        recompute = 0
        if mem(0) > limit:
            # greedy, largest-activation first == whole layers, all equal here (reference :1037-1109)
            lo, hi = 0, num_layers
            if mem(num_layers) > limit:
                return None
            while lo < hi:
                mid = (lo + hi) // 2
                if mem(mid) <= limit:
                    hi = mid
                else:
                    lo = mid + 1
            recompute = lo
        time = fwd + bwd + recompute * g["layer"]["fwd"]
        db = self.profiles[choice.gpu_type]
        if not o.tp_comm_in_op_time and choice.tp > 1:
            # 2 forward + 2 backward reductions of the hidden state per layer
            ar = db.collective_ms("all_reduce", choice.tp, layer_in) * 1e3
            time += 4 * num_layers * ar
        if next_choice is not None:
            out_mb = g["layer"]["out"] if num_layers else g["pre"]["out"]
            send_mb = out_mb
            if o.comm_revised:
                nxt = self._groups(next_choice.gpu_type, mbs // next_choice.dp if mbs % next_choice.dp == 0 else local,
                                   next_choice.tp)
                if nxt is not None:
                    send_mb = max(out_mb, nxt["layer"]["in"])
            # forward activation + backward gradient
            time += 2 * db.p2p_ms(send_mb, inter_node) * 1e3
        return StageEval(time, fwd, bwd, mem(recompute), recompute, weights)

    # ------------------------------------------------------------------ op-granular stage
    def stage_eval_ops(self, stage, mbs: int, stages_behind: int, next_stage=None, inter_node: bool = False,
                       plan_recompute: bool = True) -> Optional["OpStageEval"]:
        """Cost of a `StagePlan` (any op range). Recomputation is planned per op when the stage does
        not fit: ops are marked in order of decreasing stored activation until the stage fits
        (embedding, the first LayerNorm of a layer and the tail ops are never recomputed), then
        un-marked again, cheapest recompute per MB first, while it still fits (reference:
        check_recompute, cost_model.py:1037-1109, 1224-1251). None = infeasible."""
        from .model_ops import NEVER_RECOMPUTE_OPS
        from .state import OPS_PER_LAYER as OPL, op_position
        if mbs % stage.dp:
            return None
        rows = self.op_rows(stage.gpu_types, mbs // stage.dp, stage.tp, getattr(stage, "algo", 0))
        if rows is None:
            return None
        row_of = {"pre": lambda k: rows[0], "layer": lambda k: rows[1 + k], "post": lambda k: rows[1 + OPL + k]}
        ops = []
        for i in range(stage.op_begin, stage.op_end):
            kind, k = op_position(i, self.num_layers)
            ops.append(row_of[kind](k))
        o = self.opt
        weights = sum(r.weights_mb for r in ops)
        state_mb = weights / o.bytes_per_param * (o.bytes_per_param + o.grad_bytes_per_param + o.optimizer_bytes_per_param)
        peak = max(max(r.fwd_reserved_mb, r.bwd_reserved_mb) for r in ops)
        inflight = stages_behind + 1
        limit = self.memory_limit_mb(stage.gpu_types)
        mask = list(stage.mask())

        def memory(m):
            kept = sum(r.activations_mb for r, bit in zip(ops, m) if not bit)
            # a recomputed run keeps its first input and needs room to rebuild its largest member
            kept += sum(ops[j].input_mb for j, bit in enumerate(m) if bit and (j == 0 or not m[j - 1]))
            transient = max((r.activations_mb for r, bit in zip(ops, m) if bit), default=0.0)
            return state_mb + kept * inflight + transient + peak

        if plan_recompute and memory(mask) > limit:
            free = [j for j, r in enumerate(ops) if r.name not in NEVER_RECOMPUTE_OPS and not mask[j]]
            for j in sorted(free, key=lambda j: -ops[j].activations_mb):
                mask[j] = 1
                if memory(mask) <= limit:
                    break
            if memory(mask) > limit:
                return None
            marked = [j for j in free if mask[j]]
            for j in sorted(marked, key=lambda j: -(ops[j].fwd_us / max(ops[j].activations_mb, 1e-9))):
                mask[j] = 0
                if memory(mask) > limit:
                    mask[j] = 1
        elif memory(mask) > limit:
            return None
        fwd, bwd = sum(r.fwd_us for r in ops), sum(r.bwd_us for r in ops)
        time = fwd + bwd + sum(r.fwd_us for r, bit in zip(ops, mask) if bit)
        db = self.profiles[stage.gpu_types[0]]
        if not o.tp_comm_in_op_time and stage.tp > 1:
            reductions = sum(1 for r in ops if r.name in ("enc-attention-dense", "enc-MLP-GEMM-2", "enc-attention-qkv",
                                                          "enc-MLP-GEMM-1"))
            time += reductions * db.collective_ms("all_reduce", stage.tp, rows[1].input_mb) * 1e3
        send_mb = 0.0
        if next_stage is not None:
            send_mb = self.boundary_mb(stage.op_end, rows)
            if o.comm_revised and mbs % next_stage.dp == 0:
                nxt = self.op_rows(next_stage.gpu_types, mbs // next_stage.dp, next_stage.tp)
                if nxt is not None:
                    send_mb = max(send_mb, self.boundary_mb(stage.op_end, nxt))
            time += 2 * db.p2p_ms(send_mb, inter_node) * 1e3      # forward activation + backward gradient
        return OpStageEval(time, fwd, bwd, memory(mask), tuple(mask), weights, limit, send_mb)

    def boundary_mb(self, cut: int, rows) -> float:
        """Size of what crosses a stage boundary placed before global op `cut`: the output of the op
        before it, plus the residual that is still alive when the cut falls inside a sub-block."""
        from .state import OPS_PER_LAYER as OPL, op_position
        kind, k = op_position(cut - 1, self.num_layers)
        last = rows[0] if kind == "pre" else rows[1 + k] if kind == "layer" else rows[1 + OPL + k]
        residual_alive = kind == "layer" and k not in (4, 9)      # not right after a dropout-add op
        return last.output_mb + (rows[1].input_mb if residual_alive else 0.0)

    # ------------------------------------------------------------------ pipeline / plan
    @staticmethod
    def pipeline_time_us(stage_times: Sequence[float], num_microbatches: int) -> float:
        """1F1B: max_i (t_i * (n - 1)) + sum_j t_j  (reference :799-805)."""
        return max(stage_times) * (num_microbatches - 1) + sum(stage_times)

    def grad_sync_us(self, weights_mb: float, replicas: int, gpu_type: str) -> float:
        """Exposed time of the block-wise gradient all-reduce of one stage's gradients."""
        if not self.opt.include_grad_sync or replicas <= 1:
            return 0.0
        grad_mb = weights_mb / self.opt.bytes_per_param * self.opt.grad_bytes_per_param
        db = self.profiles[gpu_type]
        n = min(8, replicas)
        ms = db.collective_ms("all_reduce", n if (("all_reduce", n) in db.collective) else 2, grad_mb)
        if ms == 0.0:
            # alpha-beta fallback from the P2P table: ring all-reduce moves 2 (n-1)/n of the data
            ms = db.p2p_ms(grad_mb * 2 * (replicas - 1) / replicas)
        return ms * 1e3 * (1.0 - self.opt.grad_sync_overlap)
