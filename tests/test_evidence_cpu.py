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
