"""Search-space features beyond the layer-boundary DP: cuts inside a layer found by the multi-hop
local search, device placement by node-order permutation, max-over-types costing of mixed stages,
the domination bound, the op-granular recompute planner, and the ranking output."""
import json
import os
import time

import pytest

from eth_b200.contract.config import normalize_flexpipe_config
from eth_b200.search import search as S
from eth_b200.search.actions import migrate_ops
from eth_b200.search.cost_model import CostModel, CostOptions, StageChoice
from eth_b200.search.device_groups import ThroughputBounds, dominates, node_orders
from eth_b200.search.profile_db import ProfileDB
from eth_b200.search.refine import Refiner
from eth_b200.search.state import PipelinePlan, StagePlan, legal_cuts, plan_from_layers, total_ops
from eth_b200.search.synthetic_profile import generate

MBS = (1, 2, 4, 8)


@pytest.fixture(scope="module")
def two_types(tmp_path_factory):
    """Profile view with a fast and a 2.5x slower GPU type: <root>/<type>/gpt_1_3B/..."""
    root = tmp_path_factory.mktemp("view")
    for name, slow in (("fast-gpu", 1.0), ("slow-gpu", 2.5)):
        d = root / name / "gpt_1_3B"
        generate(str(d), "1_3B", name, (1, 2, 4), seed=0, slowdown=slow)
        os.replace(d / "p2p_intra_node.csv", root / name / "p2p_intra_node.csv")
    return root


def _cost(root, layers, memory=64000.0):
    profiles = {t: ProfileDB.load(str(root / t / "gpt_1_3B"), t, "1_3B", MBS, 4, p2p_dir=str(root / t))
                for t in ("fast-gpu", "slow-gpu")}
    return CostModel(profiles, layers, {t: memory for t in profiles}, CostOptions())


def test_legal_cuts_by_grain():
    assert legal_cuts(2, "layer") == [11]
    assert legal_cuts(2, "block") == [6, 11, 16]
    assert legal_cuts(2, "op") == list(range(1, total_ops(2)))


def test_migration_passes_work_through_intermediate_stages():
    plan = plan_from_layers([2, 2, 2], [(1, 1, 1, ("fast-gpu",))] * 3, 4, 6)
    moved = list(migrate_ops(plan, 0, 2, 6, "layer", max_steps=1))[0]
    sizes = [s.num_ops for s in moved.stages]
    assert sizes == [plan.stages[0].num_ops - 10, plan.stages[1].num_ops, plan.stages[2].num_ops + 10]


def test_mid_layer_cut_beats_the_layer_boundary_optimum(two_types):
    """Three layers on two equal GPUs: whole layers can only be split 2 + 1; cutting inside the
    middle layer balances the stages, and only the op-grain local search can find that."""
    layers = 3
    cost = _cost(two_types, layers)
    deadline = time.time() + 20

    def solve(grain):
        refiner = Refiner(cost, layers, grain, MBS, 4, 16, 2048, max_hops=4) if grain else None
        searcher = S.PipelineSearcher(cost, layers, 4, [4], 16, 2048, deadline, refiner=refiner, refine_seconds=5.0)
        return searcher.best(("fast-gpu", "fast-gpu"), (2, 2), 2)[4]

    by_layer, by_op = solve(None), solve("op")
    assert by_layer.op_counts is None and sorted(by_layer.layers) == [1, 2]
    assert by_op.found_by == "multi-hop" and by_op.bottleneck_us < 0.93 * by_layer.bottleneck_us
    first_stage_ops = by_op.op_counts[0]
    assert (first_stage_ops - 1) % 10 != 0                      # the cut is inside a layer
    # the op-granular result is a valid public config
    pipe = S.pipeline_to_pipe_dict(by_op, 64, layers)
    cfg = S.make_config([pipe], num_layers=layers, hidden_size=2048, num_attention_heads=16, seq_length=2048)
    assert normalize_flexpipe_config(cfg)["pipe"][0]["num_ops_in_each_stage"] == by_op.op_counts


def test_mixed_stage_runs_at_its_slowest_type(two_types):
    cost = _cost(two_types, 4)
    fast = cost.stage_eval(StageChoice(2, 2, 1, "fast-gpu"), 4, 0, 2, True, False, 1)
    slow = cost.stage_eval(StageChoice(2, 2, 1, "slow-gpu"), 4, 0, 2, True, False, 1)
    mixed = cost.stage_eval(StageChoice(2, 2, 1, "fast-gpu", gpu_types=("fast-gpu", "slow-gpu")), 4, 0, 2, True, False, 1)
    assert fast.time_us < slow.time_us and abs(mixed.time_us - slow.time_us) < 1e-6 * slow.time_us


def test_op_granular_recompute_planner_marks_only_what_is_needed(two_types):
    roomy, tight = _cost(two_types, 8, memory=64000.0), _cost(two_types, 8, memory=14000.0)
    stage = StagePlan(0, total_ops(8), 1, 1, 1, ("fast-gpu",))
    free, squeezed = roomy.stage_eval_ops(stage, 4, 0), tight.stage_eval_ops(stage, 4, 0)
    assert free is not None and not any(free.recompute)
    assert squeezed is not None and any(squeezed.recompute) and not all(squeezed.recompute[1:-2])
    assert squeezed.memory_mb <= squeezed.memory_limit_mb and squeezed.time_us > free.time_us
    assert squeezed.recompute[0] == 0 and squeezed.recompute[-1] == 0 and squeezed.recompute[-2] == 0   # never recomputed
    assert _cost(two_types, 8, memory=9000.0).stage_eval_ops(stage, 4, 0) is None


def test_node_orders_and_domination_bound():
    nodes = [{"GPU": "a", "GPU_NUM": 2}, {"GPU": "b", "GPU_NUM": 2}, {"GPU": "a", "GPU_NUM": 2}, {"GPU": "b", "GPU_NUM": 2}]
    orders = node_orders(nodes)
    assert orders[0] == (0, 1, 2, 3) and len(orders) == 6          # 4! / (2! 2!) distinct kind sequences
    kinds = {tuple(nodes[i]["GPU"] for i in o) for o in orders}
    assert ("a", "a", "b", "b") in kinds and len(kinds) == 6
    assert node_orders(nodes[:1] * 3) == [(0, 1, 2)]
    assert dominates([(2, 80), (2, 80), (1, 40)], [(1, 40), (2, 60)])
    assert not dominates([(2, 80), (1, 40)], [(2, 60), (2, 60)])
    tb = ThroughputBounds({"a": 2.0, "b": 1.0}, {"a": 80.0, "b": 80.0})
    tb.record(("a", "a"), 5.0)
    assert tb.upper_bound(("a", "b")) == 5.0 and tb.upper_bound(("b",)) == 5.0
    assert tb.upper_bound(("a", "a", "a")) == float("inf")


def _search(two_types, tmp_path, name, extra):
    out = tmp_path / name
    node_info = {"0": {"GPU": "fast-gpu", "GPU_NUM": 2, "NODE_NUM": 1}, "1": {"GPU": "slow-gpu", "GPU_NUM": 2, "NODE_NUM": 1},
                 "2": {"GPU": "fast-gpu", "GPU_NUM": 2, "NODE_NUM": 1}, "3": {"GPU": "slow-gpu", "GPU_NUM": 2, "NODE_NUM": 1}}
    device = tmp_path / "device.json"
    device.write_text(json.dumps({"fast-gpu": {"memory": 64000, "intra_bandwidth": 20, "TFLOPS": 250},
                                  "slow-gpu": {"memory": 64000, "intra_bandwidth": 20, "TFLOPS": 100}}))
    argv = ["--model-size", "1_3B", "--global-batch-size", "256", "--micro-batch-size", "1", "2", "4", "8",
            "--node-info", json.dumps(node_info), "--device-json-path", str(device), "--profiled-time-path", str(two_types),
            "--config-save-path", str(out), "--max-tp", "4", "--time-budget-total", "25", "--homo-stage", "--use-cache",
            "--sort-pipeline", "--optimal-prune", "--reduce-output", "--end-num-stages", "4", "--max-num-pipeline", "2",
            "--num-of-saved-configs", "3"] + extra
    plan, summary = S.main(argv)
    return plan, summary, out


def test_permuted_placement_wins_on_a_two_type_cluster(two_types, tmp_path):
    """Nodes arrive interleaved fast / slow. With the given order every contiguous pipeline mixes
    fast and slow stages; regrouping the nodes by type gives homogeneous pipelines that the batch
    balancer can load in proportion to their speed."""
    fixed, s_fixed, _ = _search(two_types, tmp_path, "fixed", ["--no-permute-nodes"])
    free, s_free, out = _search(two_types, tmp_path, "free", [])
    assert s_fixed["node_order"] == [0, 1, 2, 3] and s_free["node_orders"] > 1
    assert s_free["iteration_ms"] < 0.999 * s_fixed["iteration_ms"], (s_free["iteration_ms"], s_fixed["iteration_ms"])
    assert s_free["node_order"] != [0, 1, 2, 3]
    # ranking: up to three distinct plans, best first, plus the trend of improvements
    ranked = sorted(os.listdir(out / "top_configs"))
    assert ranked[0] == "eth_gpt_hybrid.json" and 1 <= len(ranked) <= 3
    rows = (out / "csv" / "eth_gpt_ranking.csv").read_text().strip().splitlines()
    times = [float(r.split(",")[1]) for r in rows[1:]]
    assert times == sorted(times) and len(times) == len(ranked)
    assert (out / "csv" / "eth_gpt_trend.csv").read_text().count("\n") >= 2
    normalize_flexpipe_config(json.loads((out / "top_configs" / "eth_gpt_hybrid.json").read_text()))


def test_swapped_sharding_is_chosen_where_the_profile_says_it_is_faster(tmp_path):
    """A profile whose algo-1 GEMM rows are much cheaper at TP2: the local search flips the stage to
    algo 1, and the serialised plan carries algo 1 with resharding enabled for that stage."""
    import csv
    d = tmp_path / "fast-gpu" / "gpt_1_3B"
    generate(str(d), "1_3B", "fast-gpu", (1, 2), seed=0)
    os.replace(d / "p2p_intra_node.csv", tmp_path / "fast-gpu" / "p2p_intra_node.csv")
    gemms = ("enc-attention-qkv", "enc-attention-dense", "enc-MLP-GEMM-1", "enc-MLP-GEMM-2")
    for mbs in MBS:
        path = d / f"gpt_1_3B_mbs{mbs}_tp2_algo1.csv"
        rows = list(csv.reader(open(path)))
        for r in rows[1:]:
            if r[0] in gemms:
                r[1], r[2] = f"{float(r[1]) * 0.4:.3f}", f"{float(r[2]) * 0.4:.3f}"
        csv.writer(open(path, "w", newline="")).writerows(rows)
    layers = 2
    profiles = {"fast-gpu": ProfileDB.load(str(d), "fast-gpu", "1_3B", MBS, 2, p2p_dir=str(tmp_path / "fast-gpu"))}
    cost = CostModel(profiles, layers, {"fast-gpu": 64000.0}, CostOptions())
    refiner = Refiner(cost, layers, "layer", MBS, 2, 16, 2048, max_hops=3, allow_exchange=False)
    start = plan_from_layers([layers], [(2, 2, 1, ("fast-gpu",))], 4, layers)
    best = refiner.refine(start, time.time() + 10)
    assert best.plan.stages[0].algo == 1 and best.per_sample_us() < refiner.score(start).per_sample_us()
    searcher = S.PipelineSearcher(cost, layers, 2, [4], 16, 2048, time.time() + 10, refiner=refiner)
    result = searcher._from_scored(best, "multi-hop")
    pipe = S.pipeline_to_pipe_dict(result, 64, layers)
    assert pipe["algo_of_each_op"] == [[1] * total_ops(layers)] and pipe["resharding_stages"] == [True]
    cfg = S.make_config([pipe], num_layers=layers, hidden_size=2048, num_attention_heads=16, seq_length=2048)
    assert normalize_flexpipe_config(cfg)["pipe"][0]["algo_of_each_op"][0][0] == 1
    # and it round-trips as a start point
    assert searcher._to_plan(result).stages[0].algo == 1


def test_multi_process_search_finds_the_same_plan(two_types, tmp_path):
    """Device groups solved in worker processes, combined by the driver: same plan, same config hash
    as the single-process search, and the driver itself evaluates no pipeline."""
    one, s_one, _ = _search(two_types, tmp_path, "one", [])
    many, s_many, _ = _search(two_types, tmp_path, "many", ["--multi-process", "--num-multi-process", "3"])
    assert s_many["config_hash"] == s_one["config_hash"]
    assert abs(s_many["iteration_ms"] - s_one["iteration_ms"]) < 1e-9
    mp = s_many["multi_process"]
    assert mp["processes"] == 3 and mp["device_groups"] >= 4
    assert mp["evaluated"] == s_many["pipelines_evaluated"] > 0        # every evaluation happened in a worker
    assert S.plan_signature(many) == S.plan_signature(one)
