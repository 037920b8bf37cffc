"""Numerical evidence: per-rank snapshots of logical parameters, gradients and optimizer state at
named phases, and reconstruction of full logical tensors from snapshots taken under any layout.

Protocol (reference: eth/runtime/megatron/grad_sync/evidence.py:158-253 snapshots, :275-415
reconstruction, :418-507 reference computations): a run with `--grad-sync-evidence-dir` writes
`rank-<r>/iter-<i>-<phase>.pt` for phase in {init, pre_sync, post_sync, post_step}; two runs under
different topologies must reconstruct to the same logical tensors, and a one-rank run over the
same global batch is the oracle (`tools/validation/compare_numerical_evidence.py`).
"""
from __future__ import annotations

import hashlib
import math
import os
from typing import Dict, Iterable, List, Tuple

import torch

PHASES = ("init", "pre_sync", "post_sync", "post_step")


def logical_seed(logical_id: str) -> int:
    return int.from_bytes(hashlib.sha256(logical_id.encode()).digest()[:8], "little") & ((1 << 63) - 1)


def canonical_logical_tensor(logical_id: str, full_shape, low=-0.02, high=0.02) -> torch.Tensor:
    """Deterministic U(low, high) tensor seeded by the logical id (layout independent)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(logical_seed(logical_id))
    return torch.rand(tuple(full_shape), generator=g, dtype=torch.float32) * (high - low) + low


def snapshot_rank(engine, phase: str, iteration: int, out_dir: str, extra=None) -> str:
    if phase not in PHASES:
        raise ValueError(f"unknown evidence phase {phase!r}")
    ps = engine.pstate
    records = []
    opt = engine.optimizer
    for e in engine.stage.unique_entries():
        st = opt.state_for_model_parameter(e.param)
        records.append({
            "logical_param_id": e.spec.logical_id, "full_shape": tuple(e.spec.full_shape),
            "partition_dim": e.spec.partition_dim, "partition_stride": e.spec.partition_stride,
            "tp_degree": ps.tp_size, "tp_rank": ps.tp_rank, "dp_rank": ps.dp_rank, "pipeline_id": ps.pipeline_id,
            "stage_id": ps.stage_id, "weight_decay": bool(e.spec.weight_decay),
            "param": e.param.detach().float().cpu(),
            "main_grad": e.param.main_grad.detach().float().cpu(),
            "master": st.get("master", e.param).detach().float().cpu(),
            "exp_avg": st["exp_avg"].detach().cpu(), "exp_avg_sq": st["exp_avg_sq"].detach().cpu()})
    loss_scale = engine.scaler.value() if engine.scaler is not None else 1.0
    payload = {"version": 2, "global_rank": engine.args.rank, "phase": phase, "iteration": iteration,
               "records": records, "metrics": dict(extra or {}), "lr": opt.lr, "step_count": opt.step_count,
               "loss_scale": loss_scale,
               "clock": {"learning_rate": opt.lr, "global_data_cursor": engine.clock.global_data_cursor,
                         "successful_optimizer_steps": engine.clock.successful_optimizer_steps,
                         "loss_scale": loss_scale},
               "run": run_metadata(engine)}
    d = os.path.join(out_dir, f"rank-{engine.args.rank:05d}")
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"iter-{iteration:05d}-{phase}.pt")
    torch.save(payload, path)
    return path


def run_metadata(engine) -> dict:
    """What an offline checker needs to re-derive an iteration: batch and loss normalisation,
    clipping, the optimizer's hyper-parameters, the learning-rate schedule, the loss-scale mode."""
    a, opt, sched = engine.args, engine.optimizer, engine.lr_scheduler
    dynamic = engine.scaler is not None and getattr(a, "loss_scale", None) is None
    return {"total_gbs": int(a.total_gbs), "nominal_global_loss_scale": float(a.nominal_global_loss_scale),
            "clip_grad": float(a.clip_grad), "optimizer": getattr(a, "optimizer", "adam"),
            "beta1": float(getattr(a, "adam_beta1", 0.9)), "beta2": float(getattr(a, "adam_beta2", 0.999)),
            "eps": float(getattr(a, "adam_eps", 1e-8)), "weight_decay": float(getattr(a, "weight_decay", 0.0)),
            "lr": sched.max_lr, "min_lr": sched.min_lr, "lr_warmup_samples": int(sched.warmup_steps),
            "lr_decay_samples": int(sched.decay_steps), "lr_decay_style": sched.decay_style,
            "loss_scale_mode": "none" if engine.scaler is None else ("dynamic" if dynamic else "static"),
            "world_size": int(a.world_size)}


def load_snapshots(run_dir: str, iteration: int, phase: str) -> List[dict]:
    out = []
    for name in sorted(os.listdir(run_dir)):
        p = os.path.join(run_dir, name, f"iter-{iteration:05d}-{phase}.pt")
        if name.startswith("rank-") and os.path.exists(p):
            out.append(torch.load(p, weights_only=False))
    if not out:
        raise FileNotFoundError(f"no snapshots for iteration {iteration} phase {phase} in {run_dir}")
    return out


def shard_intervals(size: int, tp: int, rank: int, stride: int):
    chunk = size // (tp * stride)
    return [((b * tp + rank) * chunk, (b * tp + rank + 1) * chunk) for b in range(stride)]


def reconstruct(snapshots: Iterable[dict], field: str, pipeline_id: int = 0, dp_rank: int = 0) -> Dict[str, torch.Tensor]:
    """Full logical tensors of `field` from the shards of one (pipeline, DP) replica."""
    pieces: Dict[str, list] = {}
    for snap in snapshots:
        for r in snap["records"]:
            if r["pipeline_id"] == pipeline_id and r["dp_rank"] == dp_rank:
                pieces.setdefault(r["logical_param_id"], []).append(r)
    out = {}
    for lid, recs in pieces.items():
        ref = recs[0]
        if ref["partition_dim"] < 0 or ref["tp_degree"] == 1:
            out[lid] = recs[0][field]
            continue
        axis, tp, stride = ref["partition_dim"], ref["tp_degree"], ref["partition_stride"]
        full = torch.empty(ref["full_shape"], dtype=recs[0][field].dtype)
        seen = set()
        for r in recs:
            if r["tp_rank"] in seen:
                continue   # a tied weight held by two stages: identical copies
            seen.add(r["tp_rank"])
            off = 0
            for b, e in shard_intervals(ref["full_shape"][axis], tp, r["tp_rank"], stride):
                full.narrow(axis, b, e - b).copy_(r[field].narrow(axis, off, e - b))
                off += e - b
        if seen != set(range(tp)):
            raise ValueError(f"missing TP shards of {lid}: have {sorted(seen)} of {tp}")
        out[lid] = full
    return out


def replicas(snapshots: Iterable[dict]) -> List[Tuple[int, int]]:
    return sorted({(r["pipeline_id"], r["dp_rank"]) for s in snapshots for r in s["records"]})


def max_relative_difference(a: Dict[str, torch.Tensor], b: Dict[str, torch.Tensor]) -> Tuple[float, str]:
    worst, where = 0.0, ""
    if set(a) != set(b):
        raise ValueError(f"logical parameter sets differ: {sorted(set(a) ^ set(b))[:4]}")
    for k in a:
        if a[k].shape != b[k].shape:
            raise ValueError(f"shape mismatch for {k}: {tuple(a[k].shape)} vs {tuple(b[k].shape)}")
        d = (a[k].double() - b[k].double()).norm().item() / (b[k].double().norm().item() + 1e-30)
        if d > worst:
            worst, where = d, k
    return worst, where


def reference_clip_coefficient(grads: Dict[str, torch.Tensor], max_norm: float) -> Tuple[float, float]:
    total = math.sqrt(sum(float(g.double().pow(2).sum()) for g in grads.values()))
    return total, min(1.0, max_norm / (total + 1.0e-6)) if max_norm > 0 else 1.0


def adamw_reference_step(param, grad, exp_avg, exp_avg_sq, step, lr, beta1, beta2, eps, weight_decay):
    """One decoupled-weight-decay Adam step in fp64 (reference: evidence.py:476-507)."""
    p, g = param.double(), grad.double()
    m = exp_avg.double() * beta1 + (1 - beta1) * g
    v = exp_avg_sq.double() * beta2 + (1 - beta2) * g * g
    p = p * (1 - lr * weight_decay)
    denom = v.sqrt() / math.sqrt(1 - beta2 ** step) + eps
    p = p - lr / (1 - beta1 ** step) * m / denom
    return p, m, v


# ------------------------------------------------------------------------------------------
# references that need every holder of a parameter, not one replica
# ------------------------------------------------------------------------------------------
def holders(snapshots: Iterable[dict]) -> List[Tuple[int, int, int]]:
    """Every (pipeline, DP rank, stage) that holds parameters. A tied weight has two holders in one
    replica (the embedding stage and the head stage), pipelines with different layouts hold the
    same logical parameters under different TP degrees."""
    return sorted({(r["pipeline_id"], r["dp_rank"], r["stage_id"]) for s in snapshots for r in s["records"]})


def reconstruct_holder(snapshots: Iterable[dict], field: str, holder: Tuple[int, int, int]) -> Dict[str, torch.Tensor]:
    """Full logical tensors of `field` from the shards one holder's TP ranks wrote, each record
    laid out by its own (tp_degree, partition_dim, stride): holders may disagree on the layout."""
    pid, dpr, stage = holder
    narrowed = [{"records": [r for r in s["records"]
                             if (r["pipeline_id"], r["dp_rank"], r["stage_id"]) == holder]} for s in snapshots]
    return reconstruct(narrowed, field, pid, dpr)


def full_gradient_reference(pre_sync: Iterable[dict]) -> Dict[str, torch.Tensor]:
    """What gradient synchronisation has to produce: for every logical parameter the sum, in fp64,
    of the full gradients of all its holders before the sync (all pipelines, all DP replicas, both
    ends of a tied weight). Reference: evidence.py:418-449 (there followed by the normalisation
    scale, which this engine applies in the optimizer instead)."""
    pre_sync = list(pre_sync)
    total: Dict[str, torch.Tensor] = {}
    for holder in holders(pre_sync):
        for lid, g in reconstruct_holder(pre_sync, "main_grad", holder).items():
            total[lid] = g.double() if lid not in total else total[lid] + g.double()
    return total


def reconstruct_agreed(snapshots: Iterable[dict], field: str, rtol: float = 0.0) -> Tuple[Dict[str, torch.Tensor], List[str]]:
    """(logical tensors, disagreements): `field` reconstructed from every holder; all holders of a
    logical parameter must agree within `rtol` (relative to the largest magnitude)."""
    snapshots = list(snapshots)
    agreed: Dict[str, torch.Tensor] = {}
    problems: List[str] = []
    for holder in holders(snapshots):
        for lid, value in reconstruct_holder(snapshots, field, holder).items():
            if lid not in agreed:
                agreed[lid] = value
                continue
            bound = rtol * float(agreed[lid].abs().max()) if rtol else 0.0
            if value.shape != agreed[lid].shape or float((value.double() - agreed[lid].double()).abs().max()) > bound:
                problems.append(f"{field} of {lid} differs at holder (pipeline, dp, stage) = {holder}")
    return agreed, problems


def compare_logical_tensors(actual: Dict[str, torch.Tensor], expected: Dict[str, torch.Tensor], rtol: float,
                            atol: float) -> dict:
    """Per-parameter report: worst absolute and relative error with their coordinates, and whether
    |actual - expected| <= atol + rtol * |expected| holds everywhere (non-finite values must match
    in kind and sign)."""
    rows = []
    for lid in sorted(set(actual) | set(expected)):
        if lid not in actual or lid not in expected:
            rows.append({"logical_param_id": lid, "passed": False,
                         "error": "missing actual" if lid not in actual else "missing expected"})
            continue
        a, e = actual[lid].detach().double().cpu(), expected[lid].detach().double().cpu()
        if a.shape != e.shape:
            rows.append({"logical_param_id": lid, "passed": False, "error": "shape mismatch",
                         "actual_shape": list(a.shape), "expected_shape": list(e.shape)})
            continue
        finite = torch.isfinite(a) & torch.isfinite(e)
        same_special = (~finite) & ((torch.isinf(a) & torch.isinf(e) & (torch.signbit(a) == torch.signbit(e)))
                                    | (torch.isnan(a) & torch.isnan(e)))
        diff = torch.where(finite, (a - e).abs(), torch.where(same_special, torch.zeros_like(a),
                                                              torch.full_like(a, float("inf"))))
        rel = diff / e.abs().clamp_min(max(atol, 1e-300))
        i_abs, i_rel = int(diff.reshape(-1).argmax()), int(rel.reshape(-1).argmax())
        where = lambda i: [int(v) for v in torch.unravel_index(torch.tensor(i), a.shape)] if a.dim() else []
        rows.append({"logical_param_id": lid, "passed": bool((diff <= atol + rtol * e.abs()).all()),
                     "max_abs_error": float(diff.reshape(-1)[i_abs]), "max_abs_index": where(i_abs),
                     "max_rel_error": float(rel.reshape(-1)[i_rel]), "max_rel_index": where(i_rel)})
    return {"passed": all(r["passed"] for r in rows), "rtol": rtol, "atol": atol, "parameters": rows}


def expected_learning_rate(run: dict, samples: int) -> float:
    """The schedule restated from the run metadata alone: linear warm-up over `lr_warmup_samples`,
    then constant, or linear / cosine decay to `min_lr` at `lr_decay_samples`."""
    top, low, warm, end = run["lr"], run["min_lr"], run["lr_warmup_samples"], run["lr_decay_samples"]
    if warm > 0 and samples <= warm:
        return top * samples / warm
    if run["lr_decay_style"] == "constant":
        return top
    if samples > end:
        return low
    progress = (samples - warm) / (end - warm)
    shape = 1.0 - progress if run["lr_decay_style"] == "linear" else 0.5 * (math.cos(math.pi * progress) + 1.0)
    return low + shape * (top - low)
