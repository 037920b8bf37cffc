#!/usr/bin/env python3
"""Offline oracle over numerical-evidence snapshots of two runs.

  compare_numerical_evidence.py --run-a DIR --run-b DIR --iterations 1 2 [--rtol 1e-4]
      every replica of both runs reconstructs to the same logical params / gradients / optimizer
      moments at every phase (different topologies, same global batch)
  --check-optimizer-step   additionally re-derive `post_step` from `post_sync` of run A with an
      fp64 clip + AdamW reference (weight decay on GEMM / embedding weights only)
  --check-overflow         a skipped iteration (non-finite gradients) must leave params and
      moments untouched between `post_sync` and `post_step`
Exit code 0 = consistent, 1 = mismatch (reference tool:
tools/validation/compare_numerical_evidence.py:168-285, 288-370, 409-581).
"""
import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from eth_b200.parallel.grad_sync import evidence as ev  # noqa: E402

FIELDS = {"init": ("param",), "pre_sync": ("param",), "post_sync": ("param", "main_grad"),
          "post_step": ("param", "master", "exp_avg", "exp_avg_sq")}


def compare_runs(run_a, run_b, iterations, rtol):
    problems = []
    for it in iterations:
        for phase, fields in FIELDS.items():
            try:
                sa, sb = ev.load_snapshots(run_a, it, phase), ev.load_snapshots(run_b, it, phase)
            except FileNotFoundError:
                continue
            for field in fields:
                ref = ev.reconstruct(sa, field, *ev.replicas(sa)[0])
                for run, snaps in (("a", sa), ("b", sb)):
                    for pid, dpr in ev.replicas(snaps):
                        got = ev.reconstruct(snaps, field, pid, dpr)
                        common = {k: got[k] for k in got if k in ref}
                        d, where = ev.max_relative_difference(common, {k: ref[k] for k in common})
                        if d > rtol:
                            problems.append(f"iter {it} {phase} {field}: run {run} pipeline {pid} dp {dpr} differs "
                                            f"by {d:.3e} at {where}")
    return problems


def decays(logical_id: str) -> bool:
    return logical_id.endswith("weight") and "layernorm" not in logical_id


def check_optimizer_step(run, iterations, rtol, args):
    problems = []
    for it in iterations:
        pre, post = ev.load_snapshots(run, it, "post_sync"), ev.load_snapshots(run, it, "post_step")
        grads = ev.reconstruct(pre, "main_grad")
        factor = pre[0]["metrics"].get("grad_factor", 1.0)
        grads = {k: v * factor for k, v in grads.items()}
        total, coef = ev.reference_clip_coefficient(grads, args.clip_grad)
        before = {f: ev.reconstruct(pre, f) for f in ("master", "exp_avg", "exp_avg_sq")}
        after = {f: ev.reconstruct(post, f) for f in ("master", "exp_avg", "exp_avg_sq")}
        step, lr = post[0]["step_count"], pre[0]["lr"]
        for k, g in grads.items():
            p, m, v = ev.adamw_reference_step(before["master"][k], g * coef, before["exp_avg"][k], before["exp_avg_sq"][k],
                                              step, lr, args.beta1, args.beta2, args.eps,
                                              args.weight_decay if decays(k) else 0.0)
            d = (p - after["master"][k].double()).norm().item() / (p.norm().item() + 1e-30)
            if d > rtol:
                problems.append(f"iter {it}: AdamW reference differs by {d:.3e} at {k} (norm {total:.4f}, clip {coef:.4f})")
    return problems


def compare_overflow_semantics(run, iterations):
    problems = []
    for it in iterations:
        pre, post = ev.load_snapshots(run, it, "post_sync"), ev.load_snapshots(run, it, "post_step")
        if post[0]["metrics"].get("update_successful", True):
            continue
        for f in ("master", "exp_avg", "exp_avg_sq"):
            a, b = ev.reconstruct(pre, f), ev.reconstruct(post, f)
            for k in a:
                if not torch.equal(a[k], b[k]):
                    problems.append(f"iter {it}: skipped step changed {f} of {k}")
    return problems


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--run-a", required=True)
    ap.add_argument("--run-b", default=None)
    ap.add_argument("--iterations", type=int, nargs="+", default=[1])
    ap.add_argument("--rtol", type=float, default=1e-4)
    ap.add_argument("--check-optimizer-step", action="store_true")
    ap.add_argument("--check-overflow", action="store_true")
    ap.add_argument("--clip-grad", type=float, default=1.0)
    ap.add_argument("--beta1", type=float, default=0.9)
    ap.add_argument("--beta2", type=float, default=0.999)
    ap.add_argument("--eps", type=float, default=1e-8)
    ap.add_argument("--weight-decay", type=float, default=0.01)
    a = ap.parse_args(argv)
    problems = []
    if a.run_b:
        problems += compare_runs(a.run_a, a.run_b, a.iterations, a.rtol)
    if a.check_optimizer_step:
        problems += check_optimizer_step(a.run_a, a.iterations, a.rtol, a)
    if a.check_overflow:
        problems += compare_overflow_semantics(a.run_a, a.iterations)
    print(json.dumps({"consistent": not problems, "problems": problems[:20]}, indent=1))
    return 1 if problems else 0


if __name__ == "__main__":
    raise SystemExit(main())
