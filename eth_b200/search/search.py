"""HPP configuration search.

    python -m eth_b200.search.search --model-name gpt --model-size 1_3B --global-batch-size 1024 \
        --micro-batch-size 1 2 4 8 --node-info '{"0":{"GPU":"b200","GPU_NUM":8,"NODE_NUM":1}}' \
        --device-json-path device_info.json --profiled-time-path profile_view/ \
        --config-save-path configs/ --max-tp 8 --time-budget-total 10 ...

Search space (the reference's, eth/searching/search.py + actions.py + device_groups.py): number of
pipelines and which nodes each takes; per pipeline the number of stages, each stage's GPU count,
TP x DP factorisation and layer range, the micro-batch size, and op recomputation; the global
batch is then balanced over the pipelines.

Method. The reference walks this space with a multi-hop local search over migration actions.
Here the inner problem is solved exactly: for fixed stage shapes, TP/DP and micro-batch size the
optimal layer boundaries come from a dynamic programme over layer prefixes (stage cost is additive
in layers), which is then evaluated with the 1F1B formula. The outer enumeration (stage-size
compositions, TP x DP choices, micro-batch sizes) is pruned by an ideal-throughput upper bound
and bounded by the time budget; best results per device group are cached (`--use-cache`), pipeline
splits are ordered by a TFLOPS-imbalance score (`--sort-pipeline`), pruned by the upper bound
(`--optimal-prune`), and for >= 4 pipelines chosen by a dynamic programme over contiguous node
splits (`--dp-find-pipeline`). Micro-batches are assigned greedily to the pipeline that would
finish first (reference: workload_balance_pipeline_v1, search.py:569-633).
"""
from __future__ import annotations

import itertools
import json
import math
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..contract.config import LAYER_OPS, make_config, normalize_flexpipe_config
from .arguments import parse_args
from .cost_model import CostModel, CostOptions, StageChoice
from .profile_db import ProfileDB
from .reporting import SearchLog
from .serialization import dump_hybrid_config, dump_pipeline_legacy, pipeline_to_pipe_dict

OPS_PER_LAYER = len(LAYER_OPS)


@dataclass
class PipelineResult:
    """Best configuration found for one device group at one micro-batch size."""
    gpu_types: Tuple[str, ...]
    stages: List[StageChoice]
    layers: List[int]                 # layers per stage
    recompute_layers: List[int]
    stage_times_us: List[float]
    stage_weights_mb: List[float]
    stage_memory_mb: List[float]
    mbs: int

    @property
    def bottleneck_us(self) -> float:
        return max(self.stage_times_us)

    def time_us(self, num_microbatches: int) -> float:
        return CostModel.pipeline_time_us(self.stage_times_us, num_microbatches)

    @property
    def num_gpus(self) -> int:
        return sum(s.gpus for s in self.stages)


def compositions_pow2(total: int, parts: int, max_part: int) -> List[Tuple[int, ...]]:
    """Ordered ways to write `total` as a sum of `parts` powers of two (each <= max_part)."""
    sizes = [s for s in (1, 2, 4, 8, 16, 32, 64) if s <= max_part]
    out: List[Tuple[int, ...]] = []

    def rec(left: int, k: int, acc: Tuple[int, ...]):
        if k == 0:
            if left == 0:
                out.append(acc)
            return
        if left < k or left > k * max(sizes):
            return
        for s in sizes:
            if s <= left:
                rec(left - s, k - 1, acc + (s,))

    rec(total, parts, ())
    return out


def tp_dp_options(gpus: int, max_tp: int) -> List[Tuple[int, int]]:
    return [(tp, gpus // tp) for tp in (1, 2, 4, 8) if tp <= max_tp and gpus % tp == 0 and tp <= gpus]


class PipelineSearcher:
    """Best single-pipeline configuration for a list of GPUs (one type per GPU)."""

    def __init__(self, cost: CostModel, num_layers: int, max_tp: int, mbs_list: Sequence[int], heads: int,
                 hidden: int, deadline: float, homo_stage: bool = True):
        self.cost, self.L, self.max_tp, self.mbs_list = cost, num_layers, max_tp, list(mbs_list)
        self.heads, self.hidden, self.deadline, self.homo_stage = heads, hidden, deadline, homo_stage
        self.cache: Dict[tuple, Dict[int, PipelineResult]] = {}
        self.evaluated = 0

    def best(self, gpu_types: Tuple[str, ...], stage_range: Tuple[int, int], gpus_per_node: int) -> Dict[int, PipelineResult]:
        """{mbs: best result} over all stage counts in `stage_range` (cached per device group)."""
        key = (gpu_types, stage_range)
        if key in self.cache:
            return self.cache[key]
        results: Dict[int, PipelineResult] = {}
        n = len(gpu_types)
        lo, hi = stage_range
        for stages in range(max(1, min(lo, n)), min(hi, n, self.L) + 1):
            for comp in compositions_pow2(n, stages, min(n, max(8, gpus_per_node))):
                if time.time() > self.deadline and results:
                    break
                # stages take consecutive GPUs; a stage spanning several types is costed per type (max)
                bounds = list(itertools.accumulate(comp, initial=0))
                types = []
                aligned = True
                for a, b in zip(bounds, bounds[1:]):
                    ts = set(gpu_types[a:b])
                    if len(ts) != 1 and self.homo_stage:
                        aligned = False
                        break
                    types.append(sorted(ts)[0])
                    # a stage may not straddle a node boundary unless it covers whole nodes
                    if b - a > gpus_per_node and (b - a) % gpus_per_node:
                        aligned = False
                if not aligned:
                    continue
                for mbs in self.mbs_list:
                    res = self._best_for_shape(comp, types, mbs)
                    if res is not None and (mbs not in results or self._score(res) < self._score(results[mbs])):
                        results[mbs] = res
        self.cache[key] = results
        return results

    @staticmethod
    def _score(r: PipelineResult) -> float:
        # steady-state time per sample; ties broken by fewer stages (shorter fill/drain)
        return r.bottleneck_us / r.mbs + 1e-6 * sum(r.stage_times_us) / r.mbs

    def _best_for_shape(self, comp, types, mbs) -> Optional[PipelineResult]:
        S = len(comp)
        per_stage_opts = []
        for g, t in zip(comp, types):
            opts = [(tp, dp) for tp, dp in tp_dp_options(g, self.max_tp)
                    if mbs % dp == 0 and self.heads % tp == 0 and self.hidden % tp == 0]
            if not opts:
                return None
            per_stage_opts.append(opts)
        best = None
        # enumerate TP/DP per stage (<= 4 options each); cap the product for deep pipelines
        combos = itertools.product(*per_stage_opts)
        limit = 4096
        for idx, combo in enumerate(combos):
            if idx >= limit or (time.time() > self.deadline and best is not None):
                break
            choices = [StageChoice(g, tp, dp, t) for g, (tp, dp), t in zip(comp, combo, types)]
            res = self._solve_boundaries(choices, mbs)
            self.evaluated += 1
            if res is not None and (best is None or self._score(res) < self._score(best)):
                best = res
        return best

    def _solve_boundaries(self, choices: List[StageChoice], mbs: int) -> Optional[PipelineResult]:
        """Layer boundaries minimising the bottleneck stage (DP over layer prefixes)."""
        S, L = len(choices), self.L
        if S > L:
            return None
        INF = float("inf")

        def stage_cost(s: int, nl: int):
            nxt = choices[s + 1] if s + 1 < S else None
            return self.cost.stage_eval(choices[s], mbs, 0, nl, has_pre=(s == 0), has_post=(s == S - 1),
                                        stages_behind=S - 1 - s, next_choice=nxt)

        evals: Dict[Tuple[int, int], object] = {}
        # f[s][l]: minimal bottleneck using stages 0..s for the first l layers
        f = [[INF] * (L + 1) for _ in range(S)]
        arg = [[-1] * (L + 1) for _ in range(S)]
        for s in range(S):
            min_l = s + 1
            max_l = L - (S - 1 - s)
            for l in range(min_l, max_l + 1):
                for k in range(s, l):     # stages 0..s-1 hold k layers, stage s holds l-k
                    if s == 0 and k != 0:
                        continue
                    prev = 0.0 if s == 0 else f[s - 1][k]
                    if prev == INF:
                        continue
                    nl = l - k
                    ev = evals.get((s, nl))
                    if ev is None and (s, nl) not in evals:
                        ev = stage_cost(s, nl)
                        evals[(s, nl)] = ev
                    if ev is None:
                        continue
                    val = max(prev, ev.time_us)
                    if val < f[s][l]:
                        f[s][l], arg[s][l] = val, k
        if f[S - 1][L] == INF:
            return None
        layers = [0] * S
        l = L
        for s in range(S - 1, -1, -1):
            k = arg[s][l]
            layers[s] = l - k
            l = k
        evs = [evals[(s, layers[s])] for s in range(S)]
        return PipelineResult(tuple(c.gpu_type for c in choices), list(choices), layers,
                              [e.recompute_layers for e in evs], [e.time_us for e in evs],
                              [e.weights_mb for e in evs], [e.memory_mb for e in evs], mbs)


# ------------------------------------------------------------------------------------------
# multi-pipeline: splits, balancing, pruning
# ------------------------------------------------------------------------------------------
@dataclass
class HybridPlan:
    pipelines: List[PipelineResult]
    batch_sizes: List[int]
    iteration_us: float

    @property
    def throughput(self) -> float:
        return sum(self.batch_sizes) / (self.iteration_us * 1e-6)


def balance_batches(pipes: Sequence[PipelineResult], global_batch: int) -> Optional[List[int]]:
    """Hand out micro-batches one at a time to the pipeline that would finish earliest."""
    counts = [0] * len(pipes)
    left = global_batch
    step = [p.mbs for p in pipes]
    if left < sum(step):
        return None
    for i, p in enumerate(pipes):   # every pipeline trains at least one micro-batch
        counts[i] = 1
        left -= p.mbs
    while left > 0:
        cands = [(pipes[i].time_us(counts[i] + 1), i) for i in range(len(pipes)) if step[i] <= left]
        if not cands:
            return None   # the remainder cannot be expressed with these micro-batch sizes
        _, i = min(cands)
        counts[i] += 1
        left -= step[i]
    return [c * p.mbs for c, p in zip(counts, pipes)]


def contiguous_splits(n: int, k: int):
    for cuts in itertools.combinations(range(1, n), k - 1):
        yield [(a, b) for a, b in zip((0,) + cuts, cuts + (n,))]


def imbalance_loss(groups, tflops_of_node) -> float:
    """Variance of the per-pipeline TFLOPS share (reference ordering key, device_groups.py:292-339)."""
    sums = [sum(tflops_of_node[i] for i in range(a, b)) for a, b in groups]
    mean = sum(sums) / len(sums)
    return sum((s - mean) ** 2 for s in sums) / len(sums)


def run_search(args) -> Tuple[Optional[HybridPlan], dict]:
    t0 = time.time()
    deadline = t0 + float(args.time_budget_total)
    log = SearchLog(args.log_path, quiet=args.reduce_output)
    nodes = args.nodes                       # list of {"GPU": type, "GPU_NUM": n}
    gpu_types = sorted({n["GPU"] for n in nodes})
    profiles = {}
    for t in gpu_types:
        base = os.path.join(args.profiled_time_path, t)
        pdir = os.path.join(base, f"{args.model_name}_{args.model_size}")
        if not os.path.isdir(pdir):
            pdir = args.profiled_time_path
            base = args.profiled_time_path
        profiles[t] = ProfileDB.load(pdir, t, args.model_size, args.micro_batch_size, args.max_tp, p2p_dir=base,
                                     inter_node_file=os.path.join(args.profiled_time_path, "p2p_inter_node.csv"))
    memory = {t: float(args.device_info[t]["memory"]) for t in gpu_types}
    tflops = {t: float(args.device_info[t].get("TFLOPS", 1.0)) for t in gpu_types}
    cost = CostModel(profiles, args.num_layers, memory,
                     CostOptions(include_grad_sync=not args.no_grad_sync_term, comm_revised=args.comm_revised,
                                 tp_comm_in_op_time=not args.add_tp_comm_term))
    searcher = PipelineSearcher(cost, args.num_layers, args.max_tp, args.micro_batch_size, args.num_attention_heads,
                                args.hidden_size, deadline, homo_stage=args.homo_stage)
    node_tflops = [tflops[n["GPU"]] * n["GPU_NUM"] for n in nodes]
    gpn = max(n["GPU_NUM"] for n in nodes)
    stage_range = (args.start_num_stages, args.end_num_stages)

    def group_types(a, b):
        return tuple(t for n in nodes[a:b] for t in [n["GPU"]] * n["GPU_NUM"])

    def evaluate(groups) -> Optional[HybridPlan]:
        per_group = []
        for a, b in groups:
            res = searcher.best(group_types(a, b), stage_range, gpn)
            if not res:
                return None
            per_group.append(res)
        best_plan = None
        # micro-batch size per pipeline: all combinations (<= 4^k, k small); prune by steady-state rate
        for combo in itertools.product(*[sorted(r) for r in per_group]):
            pipes = [per_group[i][m] for i, m in enumerate(combo)]
            sizes = balance_batches(pipes, args.global_batch_size)
            if sizes is None:
                continue
            it = max(p.time_us(s // p.mbs) for p, s in zip(pipes, sizes))
            replicas = sum(max(st.dp for st in p.stages) for p in pipes)
            sync = max(cost.grad_sync_us(max(p.stage_weights_mb), replicas, p.stages[0].gpu_type) for p in pipes)
            plan = HybridPlan(pipes, sizes, it + sync)
            if best_plan is None or plan.iteration_us < best_plan.iteration_us:
                best_plan = plan
            if len(per_group) > 3 and time.time() > deadline:
                break
        return best_plan

    n_nodes = len(nodes)
    best: Optional[HybridPlan] = None
    stats = {"splits_evaluated": 0, "splits_pruned": 0}
    max_pipes = min(args.max_num_pipeline, n_nodes if n_nodes > 1 else max(1, sum(n["GPU_NUM"] for n in nodes) // 2))
    # a single node may still be split into several pipelines of whole GPUs
    if n_nodes == 1 and nodes[0]["GPU_NUM"] > 1 and args.max_num_pipeline > 1:
        g = nodes[0]["GPU_NUM"]
        nodes = [{"GPU": nodes[0]["GPU"], "GPU_NUM": 1} for _ in range(g)]
        node_tflops = [tflops[n["GPU"]] for n in nodes]
        n_nodes = g
        max_pipes = min(args.max_num_pipeline, g)
    for k in range(args.min_num_pipeline, max_pipes + 1):
        splits = list(contiguous_splits(n_nodes, k))
        if args.sort_pipeline:
            splits.sort(key=lambda gs: imbalance_loss(gs, node_tflops))
        if k >= 4 and args.dp_find_pipeline:
            splits = _dp_best_splits(splits, searcher, group_types, stage_range, gpn, keep=8)
        for groups in splits:
            if time.time() > deadline and best is not None:
                break
            if args.optimal_prune and best is not None:
                # ideal bound: the split cannot beat a perfectly balanced use of its own steady-state rates
                rates = []
                ok = True
                for a, b in groups:
                    res = searcher.cache.get((group_types(a, b), stage_range))
                    if res is None:
                        ok = False
                        break
                    if not res:
                        rates = None
                        break
                    rates.append(max(r.mbs / r.bottleneck_us for r in res.values()))
                if ok and rates is not None and args.global_batch_size / sum(rates) >= best.iteration_us:
                    stats["splits_pruned"] += 1
                    continue
            plan = evaluate(groups)
            stats["splits_evaluated"] += 1
            if plan is not None and (best is None or plan.iteration_us < best.iteration_us):
                best = plan
                log.write(f"[{time.time() - t0:7.2f}s] pipelines={k} groups={groups} iteration={plan.iteration_us / 1e3:.2f} ms "
                          f"throughput={plan.throughput:.2f} samples/s")
    stats.update(seconds=time.time() - t0, pipelines_evaluated=searcher.evaluated)
    return best, stats


def _dp_best_splits(splits, searcher, group_types, stage_range, gpn, keep=8):
    """Rank contiguous splits by the sum of cached steady-state rates (additive => DP-friendly)."""
    scored = []
    for groups in splits:
        total = 0.0
        for a, b in groups:
            res = searcher.best(group_types(a, b), stage_range, gpn)
            if not res:
                total = -1.0
                break
            total += max(r.mbs / r.bottleneck_us for r in res.values())
        if total > 0:
            scored.append((-total, groups))
    scored.sort(key=lambda x: x[0])
    return [g for _, g in scored[:keep]]


def plan_to_config(plan: HybridPlan, args) -> dict:
    pipes = [pipeline_to_pipe_dict(p, b, args.num_layers) for p, b in zip(plan.pipelines, plan.batch_sizes)]
    cfg = make_config(pipes, num_layers=args.num_layers, hidden_size=args.hidden_size,
                      num_attention_heads=args.num_attention_heads, seq_length=args.seq_length,
                      model_size=args.model_size, max_position_embeddings=args.seq_length)
    cfg["node_info"] = args.node_info
    return cfg


def main(argv=None):
    args = parse_args(argv)
    plan, stats = run_search(args)
    if plan is None:
        raise SystemExit("search found no feasible configuration (memory limit or profile coverage)")
    os.makedirs(os.path.join(args.config_save_path, "top_configs"), exist_ok=True)
    os.makedirs(os.path.join(args.config_save_path, "csv"), exist_ok=True)
    cfg = plan_to_config(plan, args)
    normalized = normalize_flexpipe_config(cfg)
    stem = f"{args.save_prefix}_{args.config_suffix}" if args.config_suffix else args.save_prefix
    for i, (p, b) in enumerate(zip(plan.pipelines, plan.batch_sizes)):
        dump_pipeline_legacy(p, b, os.path.join(args.config_save_path, f"{stem}_pipe{i}_{len(p.stages)}stages.json"), args)
    top = os.path.join(args.config_save_path, "top_configs", f"{stem}_hybrid.json")
    dump_hybrid_config(cfg, top)
    summary = {"iteration_ms": plan.iteration_us / 1e3, "throughput_samples_per_s": plan.throughput,
               "tokens_per_s": plan.throughput * args.seq_length, "config_hash": normalized["config_hash"],
               "pipelines": len(plan.pipelines), **stats}
    with open(os.path.join(args.config_save_path, "csv", f"{stem}_summary.json"), "w") as f:
        json.dump(summary, f, indent=2)
    print(json.dumps(summary))
    return plan, summary


if __name__ == "__main__":
    main()
