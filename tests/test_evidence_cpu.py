"""Numerical and runtime evidence: snapshots from runs under two layouts agree, the fp64 AdamW
reference reproduces the optimizer step, and tensor-vs-block runtime evidence is consistent."""
import json
import os
import subprocess
import sys

import pytest

from eth_b200.contract.config import make_config, make_pipe, manifest_size
from tests.helpers.multiproc import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LAYERS = 2
N = manifest_size(LAYERS)


def _run(rank, world, pipes, out_dir, mode, rt_dir):
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    cfg = make_config(pipes, num_layers=LAYERS, hidden_size=32, num_attention_heads=4, seq_length=16)
    argv = ["--hidden-dropout", "0.0", "--device", "cpu", "--vocab-size", "96", "--make-vocab-size-divisible-by", "8",
            "--lr", "1e-2", "--lr-warmup-fraction", "0.0", "--lr-decay-style", "constant", "--grad-sync-mode", mode,
            "--grad-sync-bucket-size-mb", "1", "--grad-sync-evidence-dir", out_dir, "--grad-sync-evidence-canonical-init"]
    if rt_dir:
        argv += ["--grad-sync-runtime-evidence-dir", rt_dir]
    eng = TrainEngine(parse_args(argv, config=cfg, rank=rank, world_size=world), device="cpu")
    eng.train_step()
    eng.train_step()
    return True


def test_evidence_tools(tmp_path):
    a, b = str(tmp_path / "one"), str(tmp_path / "dp2")
    rt_t, rt_b = str(tmp_path / "rt_tensor"), str(tmp_path / "rt_block")
    run_ranks(1, _run, [make_pipe([N], [1], [1], gbs=8, mbs=4)], a, "block", None)
    run_ranks(2, _run, [make_pipe([N], [1], [2], gbs=8, mbs=4)], b, "block", rt_b)
    run_ranks(2, _run, [make_pipe([N], [1], [2], gbs=8, mbs=4)], str(tmp_path / "dp2t"), "tensor", rt_t)
    tool = os.path.join(ROOT, "tools", "validation", "compare_numerical_evidence.py")
    r = subprocess.run([sys.executable, tool, "--run-a", a, "--run-b", b, "--iterations", "1", "2",
                        "--check-optimizer-step", "--check-overflow"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert json.loads(r.stdout)["consistent"]
    tool = os.path.join(ROOT, "tools", "validation", "compare_runtime_evidence.py")
    r = subprocess.run([sys.executable, tool, "--tensor", rt_t, "--block", rt_b, "--skip-payload-hash"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


def _run_schedule(rank, world, pipes, out_dir):
    """Three steps with warm-up and cosine decay, so the clock check sees a moving learning rate."""
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    cfg = make_config(pipes, num_layers=LAYERS, hidden_size=32, num_attention_heads=4, seq_length=16)
    argv = ["--hidden-dropout", "0.0", "--device", "cpu", "--vocab-size", "96", "--make-vocab-size-divisible-by", "8",
            "--lr", "1e-2", "--min-lr", "1e-3", "--lr-warmup-iters", "2", "--lr-decay-iters", "6", "--lr-decay-style",
            "cosine", "--train-iters", "6", "--clip-grad", "0.5", "--grad-sync-mode", "block", "--grad-sync-bucket-size-mb",
            "1", "--grad-sync-evidence-dir", out_dir, "--grad-sync-evidence-canonical-init",
            "--distributed-backend", "gloo"]
    eng = TrainEngine(parse_args(argv, config=cfg, rank=rank, world_size=world), device="cpu")
    for _ in range(3):
        eng.train_step()
    return True


def test_full_gradient_reference_over_mixed_layouts(tmp_path):
    """Two pipelines with different layouts (TP2 and a single GPU) and a two-stage pipeline whose tied
    embedding has two holders: the synced gradient is the fp64 sum over all holders, the logged norm
    and clip follow from it, every step is one AdamW step, and the clock follows the schedule. A
    tampered snapshot is caught."""
    import torch
    tool = os.path.join(ROOT, "tools", "validation", "compare_numerical_evidence.py")
    hetero = str(tmp_path / "hetero")
    run_ranks(3, _run_schedule, [make_pipe([N], [2], [1], gbs=4, mbs=4), make_pipe([N], [1], [1], gbs=4, mbs=2)], hetero)
    report = tmp_path / "report.json"
    r = subprocess.run([sys.executable, tool, "--run-a", hetero, "--iterations", "1", "2", "3", "--full-gradient",
                        "--rtol", "1e-5", "--output", str(report)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    full = json.loads(report.read_text())["full_gradient"]
    assert [it["iteration"] for it in full] == [1, 2, 3]
    lrs = [it["clock_before"]["learning_rate"] for it in full] + [full[-1]["clock_after"]["learning_rate"]]
    assert lrs[0] == 0.0 and abs(lrs[1] - 5e-3) < 1e-12 and abs(lrs[2] - 1e-2) < 1e-12 and 1e-3 < lrs[3] < 1e-2
    assert all(it["clip_coefficient"] < 1.0 for it in full)                     # clipping was active
    # tied embedding: two stages of one pipeline hold it
    tied = str(tmp_path / "pp2")
    run_ranks(2, _run_schedule, [make_pipe([11, N - 11], [1, 1], [1, 1], gbs=8, mbs=4)], tied)
    r = subprocess.run([sys.executable, tool, "--run-a", tied, "--iterations", "1", "2", "--full-gradient",
                        "--rtol", "1e-5"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    # tamper: scale one synced gradient on one rank -> the tool reports it
    path = os.path.join(tied, "rank-00000", "iter-00002-post_sync.pt")
    snap = torch.load(path, weights_only=False)
    snap["records"][0]["main_grad"] *= 1.01
    torch.save(snap, path)
    r = subprocess.run([sys.executable, tool, "--run-a", tied, "--iterations", "2", "--full-gradient", "--rtol", "1e-5"],
                       capture_output=True, text=True)
    assert r.returncode == 1 and "synced gradient" in r.stdout
