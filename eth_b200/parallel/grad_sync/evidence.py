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
            "stage_id": ps.stage_id, "param": e.param.detach().float().cpu(),
            "main_grad": e.param.main_grad.detach().float().cpu(),
            "master": st.get("master", e.param).detach().float().cpu(),
            "exp_avg": st["exp_avg"].detach().cpu(), "exp_avg_sq": st["exp_avg_sq"].detach().cpu()})
    payload = {"version": 1, "global_rank": engine.args.rank, "phase": phase, "iteration": iteration,
               "records": records, "metrics": dict(extra or {}), "lr": opt.lr, "step_count": opt.step_count,
               "loss_scale": engine.scaler.value() if engine.scaler is not None else 1.0}
    d = os.path.join(out_dir, f"rank-{engine.args.rank:05d}")
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"iter-{iteration:05d}-{phase}.pt")
    torch.save(payload, path)
    return path


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
