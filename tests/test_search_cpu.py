"""CPU end-to-end: synthetic seeded profile -> search_gpt.sh -> gpt_config.json -> train_gpt.sh
--validate-only; plus unit checks of the cost model, the boundary solver and batch balancing."""
import json
import os
import subprocess
import sys

import pytest

from eth_b200.contract.config import normalize_flexpipe_config
from eth_b200.search import search as S
from eth_b200.search.cost_model import CostModel, StageChoice
from eth_b200.search.profile_db import ProfileDB
from eth_b200.search.synthetic_profile import generate

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, PYTHONPATH=ROOT)


def _node_desc(path, gpus=4, nodes=1, memory=64000):
    desc = {"node_info": {"0": {"GPU": "example-gpu", "GPU_NUM": gpus, "NODE_NUM": nodes}},
            "device_info": {"example-gpu": {"memory": memory, "intra_bandwidth": 20, "TFLOPS": 100}}}
    path.write_text(json.dumps(desc))
    return path


@pytest.fixture(scope="module")
def profile(tmp_path_factory):
    d = tmp_path_factory.mktemp("prof")
    generate(str(d), "1_3B", "example-gpu", (1, 2, 4), seed=0)
    return d


def test_search_script_end_to_end(profile, tmp_path):
    node = _node_desc(tmp_path / "node.json")
    out = tmp_path / "out"
    r = subprocess.run(["bash", os.path.join(ROOT, "scripts", "search_gpt.sh"), "--profile-dir", str(profile),
                        "--model-size", "1_3B", "--search-budget", "5", "--global-batch-size", "1024",
                        "--node-description", str(node), "--output", str(out), "--python", sys.executable],
                       capture_output=True, text=True, env=ENV)
    assert r.returncode == 0, r.stdout + r.stderr
    cfg = json.loads((out / "gpt_config.json").read_text())
    assert cfg["world_size"] == 4 and cfg["total_gbs"] == 1024 and cfg["model_impl"] == "gpt"
    derived = ("config_hash", "topology_fingerprint", "manifest", "world_size", "total_gbs", "pipeline_sample_offsets")
    again = normalize_flexpipe_config({k: v for k, v in cfg.items() if k not in derived})
    assert again["config_hash"] == cfg["config_hash"] and again["topology_fingerprint"] == cfg["topology_fingerprint"]
    r = subprocess.run(["bash", os.path.join(ROOT, "scripts", "train_gpt.sh"), "--config", str(out / "gpt_config.json"),
                        "--gpus-per-node", "4", "--num-nodes", "1", "--node-rank", "0", "--master-addr", "127.0.0.1",
                        "--master-port", "29500", "--grad-sync-mode", "block", "--validate-only", "--python", sys.executable],
                       capture_output=True, text=True, env=ENV)
    assert r.returncode == 0 and "Training inputs validated" in r.stdout, r.stdout + r.stderr


def test_search_dry_run_writes_plan_only(profile, tmp_path):
    node = _node_desc(tmp_path / "node.json")
    out = tmp_path / "out"
    r = subprocess.run(["bash", os.path.join(ROOT, "scripts", "search_gpt.sh"), "--profile-dir", str(profile),
                        "--model-size", "1_3B", "--search-budget", "5", "--global-batch-size", "1024",
                        "--node-description", str(node), "--output", str(out), "--dry-run", "--python", sys.executable],
                       capture_output=True, text=True, env=ENV)
    assert r.returncode == 0 and (out / "search_plan.txt").exists() and not (out / "gpt_config.json").exists()


def test_planned_profile_is_rejected(tmp_path):
    d = tmp_path / "planned"
    generate(str(d), "1_3B", "example-gpu", (1, 2, 4), status="planned")
    node = _node_desc(tmp_path / "node.json")
    r = subprocess.run([sys.executable, "-m", "eth_b200.search.profile_validation", "--profile-dir", str(d),
                        "--model-size", "1_3B", "--node-description", str(node), "--output", str(tmp_path / "o")],
                       capture_output=True, text=True, env=ENV)
    assert r.returncode != 0 and "planned" in r.stderr


def test_profile_script_dry_run_and_argument_checks(tmp_path):
    script = os.path.join(ROOT, "scripts", "profile_gpt.sh")
    base = ["--model", "gpt", "--model-size", "1_3B", "--hardware", "b200", "--num-nodes", "1", "--gpus-per-node", "4",
            "--node-rank", "0", "--master-addr", "127.0.0.1", "--master-port", "29500", "--python", sys.executable]
    out = tmp_path / "p"
    r = subprocess.run(["bash", script, *base, "--tp-sizes", "1,2,4", "--output", str(out), "--dry-run"],
                       capture_output=True, text=True, env=ENV)
    assert r.returncode == 0, r.stderr
    meta = json.loads((out / "profile_metadata.json").read_text())
    assert meta["profile_status"] == "planned" and meta["tp_sizes"] == [1, 2, 4] and (out / "profile_plan.txt").exists()
    r = subprocess.run(["bash", script, *base, "--tp-sizes", "1,3", "--output", str(out), "--dry-run"],
                       capture_output=True, text=True, env=ENV)
    assert r.returncode == 2 and "power of two" in r.stderr
    r = subprocess.run(["bash", script, *base, "--tp-sizes", "8", "--output", str(out), "--dry-run"],
                       capture_output=True, text=True, env=ENV)
    assert r.returncode == 2 and "exceeds" in r.stderr


def test_boundary_dp_balances_layers_and_respects_memory(profile):
    db = ProfileDB.load(str(profile), "example-gpu", "1_3B", (1, 2, 4, 8), 4)
    cost = CostModel({"example-gpu": db}, 24, {"example-gpu": 64000.0})
    searcher = S.PipelineSearcher(cost, 24, 4, [1, 2, 4, 8], heads=32, hidden=2048, deadline=float("inf"))
    res = searcher._solve_boundaries([StageChoice(1, 1, 1, "example-gpu"), StageChoice(1, 1, 1, "example-gpu")], 4)
    assert res is not None and sum(res.layers) == 24 and abs(res.layers[0] - res.layers[1]) <= 2
    # a tiny memory limit forces recomputation or infeasibility
    small = CostModel({"example-gpu": db}, 24, {"example-gpu": 9000.0})
    s2 = S.PipelineSearcher(small, 24, 4, [4], heads=32, hidden=2048, deadline=float("inf"))
    r2 = s2._solve_boundaries([StageChoice(1, 1, 1, "example-gpu"), StageChoice(1, 1, 1, "example-gpu")], 4)
    assert r2 is None or max(r2.recompute_layers) > 0


def test_batch_balancing_favours_the_faster_pipeline():
    fast = S.PipelineResult(("a",), [StageChoice(1, 1, 1, "a")], [24], [0], [100.0], [1.0], [1.0], 4)
    slow = S.PipelineResult(("a",), [StageChoice(1, 1, 1, "a")], [24], [0], [300.0], [1.0], [1.0], 4)
    sizes = S.balance_batches([fast, slow], 64)
    assert sum(sizes) == 64 and sizes[0] > sizes[1] and sizes[0] % 4 == 0
    assert S.compositions_pow2(8, 3, 8) and all(sum(c) == 8 for c in S.compositions_pow2(8, 3, 8))


def test_search_on_the_measured_b200_profile(tmp_path):
    """The profile directory measured on two B200s (examples/profiles) drives a search for that node."""
    prof = os.path.join(ROOT, "examples", "profiles", "b200_gpt_1_3B")
    node = os.path.join(ROOT, "examples", "configs", "node_b200x2.json")
    out = tmp_path / "out"
    r = subprocess.run(["bash", os.path.join(ROOT, "scripts", "search_gpt.sh"), "--profile-dir", prof,
                        "--model-size", "1_3B", "--search-budget", "5", "--global-batch-size", "128",
                        "--node-description", node, "--output", str(out), "--python", sys.executable],
                       capture_output=True, text=True, env=ENV)
    assert r.returncode == 0, r.stdout + r.stderr
    cfg = json.loads((out / "gpt_config.json").read_text())
    assert cfg["world_size"] == 2 and cfg["total_gbs"] == 128
    shipped = json.loads(open(os.path.join(ROOT, "examples", "configs", "gpt_1_3b_searched_2xb200.json")).read())
    assert cfg["config_hash"] == shipped["config_hash"]      # the search is deterministic
    # one B200 holds GPT-1.3B, so the search prefers two single-GPU pipelines over TP2 on NVLink
    assert [p["num_gpus"] for p in cfg["pipe"]] == [[1], [1]]
