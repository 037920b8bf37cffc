#!/usr/bin/env python3
"""Offline oracle over numerical-evidence snapshots of two runs.

  compare_numerical_evidence.py --run-a DIR --run-b DIR --iterations 1 2 [--rtol 1e-4]
      every replica of both runs reconstructs to the same logical params / gradients / optimizer
      moments at every phase (different topologies, same global batch)
  --check-optimizer-step   additionally re-derive `post_step` from `post_sync` of run A with an
      fp64 clip + AdamW reference (weight decay on GEMM / embedding weights only)
  --check-overflow         a skipped iteration (non-finite gradients) must leave params and
      moments untouched between `post_sync` and `post_step`
  --full-gradient          re-derive every iteration of run A from its own snapshots: the synced
      gradient must be the fp64 sum of all holders' pre-sync gradients (all pipelines and DP
      replicas under their own layouts, both ends of the tied embedding), the logged norm and clip
      coefficient must follow from it, `post_step` must be one AdamW step from the previous state,
      and the clock (learning rate from the schedule, data cursor, step count) must be the one the
      run metadata predicts
  --output FILE            write the full report as JSON
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


def _scalars(snapshots, section, expected, rtol, what, problems):
    """Every rank's `section` (clock or metrics) must carry the expected scalars."""
    for snap in snapshots:
        for key, want in expected.items():
            got = snap[section].get(key)
            if got is None or want is None:
                if got is not want:
                    problems.append(f"{what}: rank {snap['global_rank']} has {key}={got}, expected {want}")
                continue
            if abs(float(got) - float(want)) > rtol * max(abs(float(want)), 1e-12) + 1e-12:
                problems.append(f"{what}: rank {snap['global_rank']} has {key}={got}, expected {want}")


def compare_full_gradient(run, iterations, rtol, atol):
    """(problems, per-iteration reports) of the self-consistency check described under --full-gradient."""
    problems, reports = [], []
    for it in iterations:
        pre, synced = ev.load_snapshots(run, it, "pre_sync"), ev.load_snapshots(run, it, "post_sync")
        post = ev.load_snapshots(run, it, "post_step")
        before = ev.load_snapshots(run, it - 1, "post_step") if it > 1 else ev.load_snapshots(run, 1, "init")
        meta = pre[0]["run"]
        # loss normalisation: the global weight is the sum of what the ranks counted
        weight = sum(float(s["metrics"]["local_loss_weight"]) for s in pre)
        scale = meta["nominal_global_loss_scale"] / weight
        _scalars(pre, "metrics", {"global_loss_weight": weight, "normalization_scale": scale}, 1e-6, f"iter {it} pre_sync", problems)
        # the synced gradient, equal on all holders, against the sum of all holders' contributions
        expected = ev.full_gradient_reference(pre)
        actual, disagreements = ev.reconstruct_agreed(synced, "main_grad", rtol)
        problems += [f"iter {it} post_sync: {d}" for d in disagreements]
        gradient_report = ev.compare_logical_tensors(actual, expected, rtol, atol)
        problems += [f"iter {it}: synced gradient of {r['logical_param_id']} is not the sum of its holders' gradients "
                     f"({r.get('error') or 'max abs error %.3e at %s' % (r['max_abs_error'], r['max_abs_index'])})"
                     for r in gradient_report["parameters"] if not r["passed"]]
        # normalised, unscaled gradient -> norm (every logical parameter once) and clip coefficient
        factor = float(synced[0]["metrics"]["grad_factor"])
        loss_scale = float(synced[0]["clock"]["loss_scale"])
        if abs(factor - scale / loss_scale) > 1e-5 * abs(factor):
            problems.append(f"iter {it}: gradient factor {factor} is not normalisation / loss scale = {scale / loss_scale}")
        grads = {k: v * factor for k, v in expected.items()}
        norm, coef = ev.reference_clip_coefficient(grads, meta["clip_grad"])
        ok = all(s["metrics"]["update_successful"] for s in post)
        if ok:
            _scalars(post, "metrics", {"grad_norm": norm, "clip_coefficient": coef}, max(rtol, 1e-4), f"iter {it} post_step", problems)
        # one AdamW step from the previous state
        state_before = {f: ev.reconstruct_agreed(before, f)[0] for f in ("master", "exp_avg", "exp_avg_sq")}
        state_after = {f: ev.reconstruct_agreed(post, f)[0] for f in ("master", "exp_avg", "exp_avg_sq")}
        decay = {r["logical_param_id"]: r.get("weight_decay", decays(r["logical_param_id"])) for s in pre for r in s["records"]}
        lr_used = float(synced[0]["clock"]["learning_rate"])
        step = int(post[0]["step_count"])
        want = {"master": {}, "exp_avg": {}, "exp_avg_sq": {}}
        for k, g in grads.items():
            if ok:
                p, m, v = ev.adamw_reference_step(state_before["master"][k], g * coef, state_before["exp_avg"][k],
                                                  state_before["exp_avg_sq"][k], step, lr_used, meta["beta1"], meta["beta2"],
                                                  meta["eps"], meta["weight_decay"] if decay[k] else 0.0)
            else:
                p, m, v = state_before["master"][k], state_before["exp_avg"][k], state_before["exp_avg_sq"][k]
            want["master"][k], want["exp_avg"][k], want["exp_avg_sq"][k] = p, m, v
        state_reports = {}
        for f in want:
            rep = ev.compare_logical_tensors(state_after[f], want[f], max(rtol, 1e-5), atol)
            state_reports[f] = rep
            problems += [f"iter {it}: {f} of {r['logical_param_id']} is not one AdamW step from the previous state"
                         for r in rep["parameters"] if not r["passed"]]
        # the clock: what the iteration started from, and what it left behind
        done_before = int(before[0]["clock"]["successful_optimizer_steps"]) if it > 1 else 0
        gbs = meta["total_gbs"]
        start = {"learning_rate": ev.expected_learning_rate(meta, done_before * gbs), "global_data_cursor": (it - 1) * gbs,
                 "successful_optimizer_steps": done_before}
        done_after = done_before + (1 if ok else 0)
        end = {"learning_rate": ev.expected_learning_rate(meta, done_after * gbs), "global_data_cursor": it * gbs,
               "successful_optimizer_steps": done_after}
        _scalars(synced, "clock", start, 1e-9, f"iter {it} clock before the step", problems)
        _scalars(post, "clock", end, 1e-9, f"iter {it} clock after the step", problems)
        reports.append({"iteration": it, "global_loss_weight": weight, "normalization_scale": scale, "grad_norm": norm,
                        "clip_coefficient": coef, "update_successful": ok, "gradients": gradient_report,
                        "optimizer_state": state_reports, "clock_before": start, "clock_after": end})
    return problems, reports


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--run-a", required=True)
    ap.add_argument("--run-b", default=None)
    ap.add_argument("--iterations", type=int, nargs="+", default=[1])
    ap.add_argument("--rtol", type=float, default=1e-4)
    ap.add_argument("--check-optimizer-step", action="store_true")
    ap.add_argument("--check-overflow", action="store_true")
    ap.add_argument("--full-gradient", action="store_true")
    ap.add_argument("--atol", type=float, default=1e-7)
    ap.add_argument("--output", default=None)
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
    full = None
    if a.full_gradient:
        found, full = compare_full_gradient(a.run_a, a.iterations, a.rtol, a.atol)
        problems += found
    if a.output:
        Path(a.output).parent.mkdir(parents=True, exist_ok=True)
        Path(a.output).write_text(json.dumps({"consistent": not problems, "problems": problems, "full_gradient": full},
                                             indent=1, sort_keys=True) + "\n")
    print(json.dumps({"consistent": not problems, "problems": problems[:20]}, indent=1))
    return 1 if problems else 0


if __name__ == "__main__":
    raise SystemExit(main())
