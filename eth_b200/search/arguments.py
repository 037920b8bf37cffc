"""Flags of `python -m eth_b200.search.search` (reference surface: eth/searching/arguments.py:21-138;
model table :10-18; node_info expansion :224-249). Every flag that scripts/search_gpt.sh passes is
accepted, and each of them acts: the heuristic flags steer the local search that refines the exact
boundary solution (refine.py)."""
from __future__ import annotations

import argparse
import json

from ..contract.config import GPT_SIZES


def build_parser():
    p = argparse.ArgumentParser(description="HPP configuration search", allow_abbrev=False)
    g = p.add_argument_group("model")
    g.add_argument("--model-name", default="gpt", choices=["gpt", "scale-layer"], help="Model family.")
    g.add_argument("--model-size", default="1_3B", help="Model size key (350M, 1_3B, 2_6B, 6_7B, 13B, 70B).")
    g.add_argument("--num-layers", type=int, default=None, help="Override the number of layers (scale-layer).")
    g.add_argument("--global-batch-size", type=int, required=True, help="Total samples per iteration.")
    g.add_argument("--micro-batch-size", type=int, nargs="+", default=[1, 2, 4, 8], help="Candidate micro-batch sizes.")
    g = p.add_argument_group("hardware")
    g.add_argument("--node-info", type=str, required=True,
                   help='JSON {id: {"GPU": type, "GPU_NUM": gpus per node, "NODE_NUM": nodes}}.')
    g.add_argument("--device-json-path", type=str, default=None, help="JSON {type: {memory, intra_bandwidth, TFLOPS}}.")
    g.add_argument("--memory-limit", type=float, default=None, help="Override the per-GPU memory limit (MB).")
    g.add_argument("--max-tp", type=int, default=8, help="Largest tensor-parallel degree covered by the profile.")
    g = p.add_argument_group("search space")
    g.add_argument("--start-num-stages", type=int, default=1, help="Smallest pipeline depth.")
    g.add_argument("--end-num-stages", type=int, default=8, help="Largest pipeline depth.")
    g.add_argument("--min-num-pipeline", type=int, default=1, help="Smallest number of pipelines.")
    g.add_argument("--max-num-pipeline", type=int, default=100, help="Largest number of pipelines.")
    g.add_argument("--op-grain", default="layer", choices=["op", "block", "layer"], help="Stage cut granularity.")
    g.add_argument("--homo-stage", action="store_true", help="Stages may not mix GPU types.")
    g = p.add_argument_group("budget and heuristics")
    g.add_argument("--time-budget-total", type=float, default=10, help="Search budget in seconds.")
    g.add_argument("--max-num-hops", type=int, default=7,
                   help="Depth of the multi-hop local search that refines the boundary-DP optimum (0 = off).")
    g.add_argument("--initial-point", default="dp",
                   help="Extra starting point of the local search: dp (the DP optimum only), balance / balance_v1 "
                        "(equal layers per stage, TP = stage GPUs), or the path of a legacy single-pipeline JSON.")
    g.add_argument("--refine-share", type=float, default=0.25,
                   help="Fraction of the time budget that one device group may spend in the local search.")
    g.add_argument("--support-comm-predict", action="store_true", help="Use measured collective tables.")
    g.add_argument("--comm-revised", action="store_true", help="Charge max(previous output, this input) per boundary.")
    g.add_argument("--add-action-tp-dp-exchange", action="store_true",
                   help="Local search may exchange TP against DP inside a stage (the DP enumerates all TP x DP anyway).")
    g.add_argument("--no-add-action-tp-dp", action="store_true", help="Local search may not move GPUs between stages.")
    g.add_argument("--use-cache", action="store_true", help="Cache the best result per device group.")
    g.add_argument("--optimal-prune", action="store_true", help="Prune pipeline splits by an ideal-throughput bound.")
    g.add_argument("--sort-pipeline", action="store_true", help="Try balanced pipeline splits first.")
    g.add_argument("--dp-find-pipeline", action="store_true", help="Choose splits of >= 4 pipelines by dynamic programming.")
    g.add_argument("--elastic-time", action="store_true",
                   help="Local-search time a device group did not use is added to the next group's allowance.")
    g.add_argument("--no-permute-nodes", dest="permute_nodes", action="store_false",
                   help="Keep the given node order (by default distinct orderings of node kinds are tried).")
    g.add_argument("--max-node-orders", type=int, default=24, help="Cap on node orderings tried.")
    g.add_argument("--no-grad-sync-term", action="store_true", help="Ignore the gradient all-reduce in the cost model.")
    g.add_argument("--add-tp-comm-term", action="store_true",
                   help="Add tensor-parallel reductions from the collective tables (profiles taken without them).")
    g = p.add_argument_group("output")
    g.add_argument("--profiled-time-path", type=str, required=True, help="Root of the profile view.")
    g.add_argument("--config-save-path", type=str, required=True, help="Directory for generated configs.")
    g.add_argument("--log-path", type=str, default=None, help="Directory for search logs.")
    g.add_argument("--config-suffix", type=str, default="", help="Suffix of generated file names.")
    g.add_argument("--save-prefix", type=str, default="eth_gpt", help="Prefix of generated file names.")
    g.add_argument("--num-of-saved-configs", type=int, default=1, help="How many top configs to keep.")
    g.add_argument("--multi-process", action="store_true",
                   help="Solve the device groups in worker processes before combining them.")
    g.add_argument("--num-multi-process", type=int, default=4, help="Worker processes of --multi-process.")
    g.add_argument("--reduce-output", action="store_true", help="Less console output.")
    return p


def expand_nodes(node_info: dict):
    """{id: {GPU, GPU_NUM, NODE_NUM}} -> one entry per node, in id order."""
    nodes = []
    for key in sorted(node_info, key=lambda k: int(k) if str(k).isdigit() else str(k)):
        e = node_info[key]
        for _ in range(int(e.get("NODE_NUM", 1))):
            nodes.append({"GPU": e["GPU"], "GPU_NUM": int(e["GPU_NUM"])})
    return nodes


def parse_args(argv=None):
    args = build_parser().parse_args(argv)
    if args.model_size not in GPT_SIZES:
        raise SystemExit(f"unsupported --model-size: {args.model_size}")
    m = GPT_SIZES[args.model_size]
    args.num_layers = args.num_layers or m["num_layers"]
    args.hidden_size, args.num_attention_heads, args.seq_length = m["hidden_size"], m["num_attention_heads"], m["seq_length"]
    args.node_info = json.loads(args.node_info) if isinstance(args.node_info, str) else args.node_info
    args.nodes = expand_nodes(args.node_info)
    args.num_gpus = sum(n["GPU_NUM"] for n in args.nodes)
    args.gpu_type_set = sorted({n["GPU"] for n in args.nodes})
    if args.device_json_path:
        with open(args.device_json_path) as f:
            args.device_info = json.load(f)
    else:
        args.device_info = {t: {"memory": args.memory_limit or 180000, "intra_bandwidth": 900, "TFLOPS": 1} for t in args.gpu_type_set}
    if args.memory_limit:
        for t in args.device_info:
            args.device_info[t]["memory"] = args.memory_limit
    args.end_num_stages = max(args.start_num_stages, args.end_num_stages)
    return args
