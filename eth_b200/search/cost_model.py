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
from functools import lru_cache
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


@dataclass
class StageEval:
    time_us: float
    fwd_us: float
    bwd_us: float
    memory_mb: float
    recompute_layers: int
    weights_mb: float


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
    def _groups(self, gpu_type: str, mbs: int, tp: int, algo: int = 0) -> Optional[dict]:
        """Sums over the three op groups of the one-layer profile: pre (embedding), layer, post."""
        key = (gpu_type, mbs, tp, algo)
        hit = self._layer_cache.get(key)
        if hit is not None or key in self._layer_cache:
            return hit
        db = self.profiles[gpu_type]
        if not db.has(mbs, tp, algo):
            self._layer_cache[key] = None
            return None
        rows = db.records(mbs, tp, algo)
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
        g = self._groups(choice.gpu_type, local, choice.tp)
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
        limit = self.device_memory_mb[choice.gpu_type] * (1.0 - o.memory_reserve_fraction)
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
