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
Here the layer-granular inner problem is solved exactly first: for fixed stage shapes, TP/DP and micro-batch size the
optimal layer boundaries come from a dynamic programme over layer prefixes (stage cost is additive
in layers), which is then evaluated with the 1F1B formula. The outer enumeration (stage-size
compositions, TP x DP choices, micro-batch sizes) is pruned by an ideal-throughput upper bound
and bounded by the time budget; best results per device group are cached (`--use-cache`), pipeline
splits are ordered by a TFLOPS-imbalance score (`--sort-pipeline`), pruned by the upper bound
(`--optimal-prune`), and for >= 4 pipelines chosen by a dynamic programme over contiguous node
splits (`--dp-find-pipeline`). Micro-batches are assigned greedily to the pipeline that would
finish first (reference: workload_balance_pipeline_v1, search.py:569-633).

On top of that: `--op-grain op|block` (or an explicit `--initial-point`) starts the multi-hop local
search of `refine.py` from the DP optimum, which may move stage cuts inside a layer, exchange TP
against DP, move GPUs between stages and change the micro-batch size (`actions.py`, `policy.py`);
device placement is searched by permuting the node order before the contiguous splits
(`--permute-nodes`, `device_groups.node_orders`); unsolved device groups are bounded by solved
groups that dominate them (`device_groups.ThroughputBounds`); the best `--num-of-saved-configs`
plans are ranked and written with trend CSVs (`reporting.Ranking`).
"""
from __future__ import annotations

import itertools
import json
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..contract.config import LAYER_OPS, make_config, normalize_flexpipe_config
from .arguments import parse_args
from .cost_model import CostModel, CostOptions, StageChoice
from .device_groups import (ThroughputBounds, compositions_pow2, contiguous_splits, imbalance_loss,  # noqa: F401
                            node_orders)
from .profile_db import ProfileDB
from .refine import Refiner
from .reporting import Ranking, SearchLog, Timers
from .serialization import dump_hybrid_config, dump_pipeline_legacy, load_initial_plan, pipeline_to_pipe_dict
from .state import PipelinePlan, StagePlan, plan_from_layers

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
    op_counts: Optional[List[int]] = None            # ops per stage when a cut falls inside a layer
    recompute_masks: Optional[List[Tuple[int, ...]]] = None   # per-op recompute flags from the op-granular planner
    found_by: str = "boundary-dp"

    @property
    def bottleneck_us(self) -> float:
        return max(self.stage_times_us)

    def time_us(self, num_microbatches: int) -> float:
        return CostModel.pipeline_time_us(self.stage_times_us, num_microbatches)

    @property
    def num_gpus(self) -> int:
        return sum(s.gpus for s in self.stages)


def tp_dp_options(gpus: int, max_tp: int) -> List[Tuple[int, int]]:
    return [(tp, gpus // tp) for tp in (1, 2, 4, 8) if tp <= max_tp and gpus % tp == 0 and tp <= gpus]


class PipelineSearcher:
    """Best single-pipeline configuration for a list of GPUs (one type per GPU)."""

    def __init__(self, cost: CostModel, num_layers: int, max_tp: int, mbs_list: Sequence[int], heads: int,
                 hidden: int, deadline: float, homo_stage: bool = True, refiner: Optional[Refiner] = None,
                 refine_seconds: float = 0.0, elastic: bool = False, initial_point: str = "dp"):
        self.cost, self.L, self.max_tp, self.mbs_list = cost, num_layers, max_tp, list(mbs_list)
        self.heads, self.hidden, self.deadline, self.homo_stage = heads, hidden, deadline, homo_stage
        self.cache: Dict[tuple, Dict[int, PipelineResult]] = {}
        self.evaluated = 0
        # local search on top of the exact layer-boundary solution (op / block grain cuts, shape moves)
        self.refiner, self.refine_seconds, self.elastic, self.initial_point = refiner, refine_seconds, elastic, initial_point
        self.budget_pool = 0.0      # refinement time that easy groups did not use (`--elastic-time`)
        self.refined = 0

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
                    types.append(tuple(sorted(ts)))     # a mixed stage is costed per op at its slowest type
                    # a stage may not straddle a node boundary unless it covers whole nodes
                    if b - a > gpus_per_node and (b - a) % gpus_per_node:
                        aligned = False
                if not aligned:
                    continue
                for mbs in self.mbs_list:
                    res = self._best_for_shape(comp, types, mbs)
                    if res is not None and (mbs not in results or self._score(res) < self._score(results[mbs])):
                        results[mbs] = res
        if self.refiner is not None and results:
            for res in self._refined(results):
                if res.mbs not in results or self._score(res) < self._score(results[res.mbs]):
                    results[res.mbs] = res
        self.cache[key] = results
        return results

    # ------------------------------------------------------------------ local search on top of the DP
    def _to_plan(self, r: PipelineResult) -> PipelinePlan:
        shapes = [(c.gpus, c.tp, c.dp, c.types()) for c in r.stages]
        if r.op_counts:
            stages, cursor = [], 0
            for n, (g, tp, dp, types), c in zip(r.op_counts, shapes, r.stages):
                stages.append(StagePlan(cursor, cursor + n, g, tp, dp, tuple(types), algo=c.algo))
                cursor += n
            return PipelinePlan(tuple(stages), r.mbs)
        return plan_from_layers(r.layers, shapes, r.mbs, self.L)

    def _from_scored(self, scored, how: str) -> PipelineResult:
        plan = scored.plan
        choices = [StageChoice(st.gpus, st.tp, st.dp, st.gpu_types[0], gpu_types=st.gpu_types, algo=st.algo)
                   for st in plan.stages]
        counts = [st.num_ops for st in plan.stages]
        layers = [max(0, round((n - (1 if i == 0 else 0) - (2 if i == len(counts) - 1 else 0)) / OPS_PER_LAYER))
                  for i, n in enumerate(counts)]
        masks = [ev.recompute for ev in scored.evals]
        return PipelineResult(tuple(c.gpu_type for c in choices), choices, layers, [0] * len(counts),
                              [e.time_us for e in scored.evals], [e.weights_mb for e in scored.evals],
                              [e.memory_mb for e in scored.evals], plan.mbs, op_counts=counts, recompute_masks=masks,
                              found_by=how)

    def _start_plans(self, results: Dict[int, PipelineResult]) -> List[PipelinePlan]:
        starts = [self._to_plan(r) for r in results.values()]
        sample = next(iter(results.values()))
        if self.initial_point in ("balance", "balance_v1"):
            # equal layers per stage, TP = the stage's GPUs, DP = 1 (reference: config.py:425-489)
            n = len(sample.stages)
            base, extra = divmod(self.L, n)
            layers = [base + (1 if i >= n - extra else 0) for i in range(n)]
            for mbs in self.mbs_list:
                shapes = []
                for c in sample.stages:
                    tp = min(c.gpus, self.max_tp)
                    shapes.append((c.gpus, tp, c.gpus // tp, c.types()))
                if all(mbs % dp == 0 for _, _, dp, _ in shapes) and all(x > 0 for x in layers):
                    starts.append(plan_from_layers(layers, shapes, mbs, self.L))
        elif self.initial_point not in ("dp", ""):
            plan = load_initial_plan(self.initial_point, self.L, sample.gpu_types)
            if plan is not None and plan.num_gpus == sample.num_gpus:
                starts.append(plan)
        return starts

    def _refined(self, results: Dict[int, PipelineResult]) -> List[PipelineResult]:
        out = []
        starts = self._start_plans(results)
        for plan in starts:
            allowance = self.refine_seconds / max(1, len(starts)) + (self.budget_pool if self.elastic else 0.0)
            t0 = time.time()
            until = min(self.deadline, t0 + allowance)
            if until <= t0:
                break
            before = len(self.refiner.trace)
            scored = self.refiner.refine(plan, until)
            used = time.time() - t0
            if self.elastic:
                self.budget_pool = max(0.0, allowance - used)
            self.refined += 1
            if scored.feasible:
                out.append(self._from_scored(scored, "multi-hop" if len(self.refiner.trace) > before else "start"))
        return out

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
            choices = [StageChoice(g, tp, dp, t[0], gpu_types=t) for g, (tp, dp), t in zip(comp, combo, types)]
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
    node_order: Tuple[int, ...] = ()                  # device placement: order of the nodes ...
    groups: Tuple[Tuple[int, int], ...] = ()          # ... and which slice of that order each pipeline takes

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


def plan_signature(plan: "HybridPlan") -> tuple:
    return tuple((p.mbs, tuple((c.gpus, c.tp, c.dp) for c in p.stages), tuple(p.op_counts or p.layers), b)
                 for p, b in zip(plan.pipelines, plan.batch_sizes)) + (plan.node_order,)


def build_searcher(args, deadline: float, timers: Optional[Timers] = None):
    """(cost model, refiner or None, pipeline searcher, memory, tflops) for a parsed argument set:
    what the driver and every worker process of a multi-process search set up alike."""
    timers = timers or Timers()
    gpu_types = sorted({n["GPU"] for n in args.nodes})
    profiles = {}
    with timers.phase("load-profiles"):
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
    # Local search on top of the boundary DP: needed for cuts inside a layer (`--op-grain op|block`);
    # at layer grain it still explores shape moves from the requested initial point.
    refiner = None
    if args.max_num_hops > 0 and (args.op_grain != "layer" or args.initial_point not in ("dp", "")):
        refiner = Refiner(cost, args.num_layers, args.op_grain, args.micro_batch_size, args.max_tp,
                          args.num_attention_heads, args.hidden_size, max_hops=args.max_num_hops,
                          allow_gpu_moves=not args.no_add_action_tp_dp, allow_exchange=args.add_action_tp_dp_exchange)
    searcher = PipelineSearcher(cost, args.num_layers, args.max_tp, args.micro_batch_size, args.num_attention_heads,
                                args.hidden_size, deadline, homo_stage=args.homo_stage, refiner=refiner,
                                refine_seconds=float(args.time_budget_total) * args.refine_share,
                                elastic=args.elastic_time, initial_point=args.initial_point)
    return cost, refiner, searcher, memory, tflops


def search_nodes(args):
    """(nodes as searched, GPUs per node): a single node may be split into pipelines of whole GPUs."""
    base_nodes = list(args.nodes)                # list of {"GPU": type, "GPU_NUM": n}
    gpn = max(n["GPU_NUM"] for n in base_nodes)
    if len(base_nodes) == 1 and base_nodes[0]["GPU_NUM"] > 1 and args.max_num_pipeline > 1:
        base_nodes = [{"GPU": base_nodes[0]["GPU"], "GPU_NUM": 1} for _ in range(base_nodes[0]["GPU_NUM"])]
    return base_nodes, gpn


def device_groups_needed(args) -> List[Tuple[str, ...]]:
    """Every distinct device group (tuple of GPU types, in device order) that some node order and
    some contiguous split into pipelines will ask the pipeline searcher about."""
    base_nodes, _ = search_nodes(args)
    n_nodes = len(base_nodes)
    orders = node_orders(base_nodes, args.max_node_orders) if args.permute_nodes else [tuple(range(n_nodes))]
    seen, out = set(), []
    for order in orders:
        nodes = [base_nodes[i] for i in order]
        for a in range(n_nodes):
            for b in range(a + 1, n_nodes + 1):
                if n_nodes - (b - a) < args.min_num_pipeline - 1:
                    continue      # too few nodes left for the other pipelines
                g = tuple(t for n in nodes[a:b] for t in [n["GPU"]] * n["GPU_NUM"])
                if g not in seen:
                    seen.add(g)
                    out.append(g)
    return out


def _solve_groups(payload):
    """Worker of the multi-process search: solve a share of the device groups, return the cache entries."""
    args, groups, deadline = payload
    _, refiner, searcher, _, _ = build_searcher(args, deadline)
    _, gpn = search_nodes(args)
    stage_range = (args.start_num_stages, args.end_num_stages)
    solved = [(g, searcher.best(g, stage_range, gpn)) for g in groups]
    return solved, searcher.evaluated, searcher.refined, refiner.evaluated if refiner else 0


def presolve_in_processes(args, searcher, deadline: float, log) -> dict:
    """Solve all device groups in `--num-multi-process` worker processes and fill the searcher's
    cache, so that the driver loop below only combines cached results (reference: one process per
    (stage count, device group, node order), eth/searching/search.py:961-1021; here the unit is the
    device group, which is what the cache is keyed by). Largest groups first, dealt round-robin."""
    import multiprocessing
    groups = sorted(device_groups_needed(args), key=lambda g: -len(g))
    workers = max(1, min(int(args.num_multi_process), len(groups)))
    shares = [groups[i::workers] for i in range(workers)]
    stage_range = (args.start_num_stages, args.end_num_stages)
    stats = {"processes": workers, "device_groups": len(groups), "evaluated": 0, "refined": 0, "refine_evaluations": 0}
    quiet = argparse_copy(args)
    with multiprocessing.get_context("spawn").Pool(workers) as pool:
        for solved, evaluated, refined, refine_evals in pool.imap_unordered(_solve_groups, [(quiet, s, deadline) for s in shares]):
            for g, res in solved:
                searcher.cache[(g, stage_range)] = res
            stats["evaluated"] += evaluated
            stats["refined"] += refined
            stats["refine_evaluations"] += refine_evals
    log.write(f"multi-process: {len(groups)} device groups solved in {workers} processes")
    return stats


def argparse_copy(args):
    """The argument set a worker gets: the same search, nothing written from the worker."""
    import copy
    quiet = copy.copy(args)
    quiet.log_path, quiet.reduce_output = None, True
    return quiet


def run_search(args) -> Tuple[Optional[HybridPlan], dict]:
    t0 = time.time()
    deadline = t0 + float(args.time_budget_total)
    log = SearchLog(args.log_path, quiet=args.reduce_output)
    timers = Timers()
    cost, refiner, searcher, memory, tflops = build_searcher(args, deadline, timers)
    bounds = ThroughputBounds(tflops, memory)
    presolved = None
    if getattr(args, "multi_process", False) and int(getattr(args, "num_multi_process", 1)) > 1:
        with timers.phase("multi-process-presolve"):
            presolved = presolve_in_processes(args, searcher, deadline, log)
    ranking = Ranking(args.num_of_saved_configs, plan_signature)
    stage_range = (args.start_num_stages, args.end_num_stages)
    stats = {"splits_evaluated": 0, "splits_pruned": 0, "node_orders": 0}

    base_nodes, gpn = search_nodes(args)
    n_nodes = len(base_nodes)
    max_pipes = min(args.max_num_pipeline, n_nodes)

    def rate_of(results) -> float:
        return max(r.mbs / r.bottleneck_us for r in results.values())

    for order in (node_orders(base_nodes, args.max_node_orders) if args.permute_nodes else [tuple(range(n_nodes))]):
        if time.time() > deadline and ranking.best is not None:
            break
        stats["node_orders"] += 1
        nodes = [base_nodes[i] for i in order]
        node_tflops = [tflops[n["GPU"]] * n["GPU_NUM"] for n in nodes]

        def group_types(a, b, nodes=nodes):
            return tuple(t for n in nodes[a:b] for t in [n["GPU"]] * n["GPU_NUM"])

        def solve(a, b):
            with timers.phase("pipeline-search"):
                res = searcher.best(group_types(a, b), stage_range, gpn)
            if res:
                bounds.record(group_types(a, b), rate_of(res))
            return res

        def evaluate(groups) -> Optional[HybridPlan]:
            per_group = []
            for a, b in groups:
                res = solve(a, b)
                if not res:
                    return None
                per_group.append(res)
            best_plan = None
            # micro-batch size per pipeline: all combinations (<= 4^k, k small)
            with timers.phase("batch-balancing"):
                for combo in itertools.product(*[sorted(r) for r in per_group]):
                    pipes = [per_group[i][m] for i, m in enumerate(combo)]
                    sizes = balance_batches(pipes, args.global_batch_size)
                    if sizes is None:
                        continue
                    it = max(p.time_us(s // p.mbs) for p, s in zip(pipes, sizes))
                    replicas = sum(max(st.dp for st in p.stages) for p in pipes)
                    sync = max(cost.grad_sync_us(max(p.stage_weights_mb), replicas, p.stages[0].gpu_type) for p in pipes)
                    plan = HybridPlan(pipes, sizes, it + sync, node_order=tuple(order), groups=tuple(groups))
                    if best_plan is None or plan.iteration_us < best_plan.iteration_us:
                        best_plan = plan
                    if len(per_group) > 3 and time.time() > deadline:
                        break
            return best_plan

        for k in range(args.min_num_pipeline, max_pipes + 1):
            splits = list(contiguous_splits(n_nodes, k))
            if args.sort_pipeline:
                splits.sort(key=lambda gs: imbalance_loss(gs, node_tflops))
            if k >= 4 and args.dp_find_pipeline:
                splits = _dp_best_splits(splits, searcher, group_types, stage_range, gpn, keep=8)
            for groups in splits:
                if time.time() > deadline and ranking.best is not None:
                    break
                if args.optimal_prune and ranking.best is not None:
                    # The split cannot beat a perfectly balanced use of its groups' best steady-state
                    # rates; a group not solved yet is bounded by a solved group that dominates it.
                    total = sum(bounds.upper_bound(group_types(a, b)) for a, b in groups)
                    if total != float("inf") and total > 0 and args.global_batch_size / total >= ranking.best.iteration_us:
                        stats["splits_pruned"] += 1
                        continue
                plan = evaluate(groups)
                stats["splits_evaluated"] += 1
                if plan is not None and ranking.offer(plan):
                    log.write(f"[{time.time() - t0:7.2f}s] node order={list(order)} pipelines={k} groups={groups} "
                              f"iteration={plan.iteration_us / 1e3:.2f} ms throughput={plan.throughput:.2f} samples/s")
    stats.update(seconds=time.time() - t0, pipelines_evaluated=searcher.evaluated, groups_refined=searcher.refined,
                 refine_evaluations=refiner.evaluated if refiner else 0, timers=timers.report())
    if presolved is not None:
        stats["multi_process"] = presolved
        stats["pipelines_evaluated"] += presolved["evaluated"]
        stats["groups_refined"] += presolved["refined"]
        stats["refine_evaluations"] += presolved["refine_evaluations"]
    stats["ranking"] = ranking
    return ranking.best, stats


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
    ranking: Ranking = stats.pop("ranking")
    os.makedirs(os.path.join(args.config_save_path, "top_configs"), exist_ok=True)
    os.makedirs(os.path.join(args.config_save_path, "csv"), exist_ok=True)
    stem = f"{args.save_prefix}_{args.config_suffix}" if args.config_suffix else args.save_prefix
    for i, (p, b) in enumerate(zip(plan.pipelines, plan.batch_sizes)):
        dump_pipeline_legacy(p, b, os.path.join(args.config_save_path, f"{stem}_pipe{i}_{len(p.stages)}stages.json"), args)
    normalized = None
    for rank, (_, ranked) in enumerate(ranking.entries, 1):
        cfg = plan_to_config(ranked, args)
        norm = normalize_flexpipe_config(cfg)
        name = f"{stem}_hybrid.json" if rank == 1 else f"{stem}_hybrid_rank{rank}.json"
        dump_hybrid_config(cfg, os.path.join(args.config_save_path, "top_configs", name))
        normalized = normalized or norm
    ranking.write_csvs(os.path.join(args.config_save_path, "csv"), stem)
    summary = {"iteration_ms": plan.iteration_us / 1e3, "throughput_samples_per_s": plan.throughput,
               "tokens_per_s": plan.throughput * args.seq_length, "config_hash": normalized["config_hash"],
               "pipelines": len(plan.pipelines), "node_order": list(plan.node_order),
               "pipeline_node_slices": [list(g) for g in plan.groups],
               "found_by": [p.found_by for p in plan.pipelines], "op_grain": args.op_grain, **stats}
    with open(os.path.join(args.config_save_path, "csv", f"{stem}_summary.json"), "w") as f:
        json.dump(summary, f, indent=2)
    print(json.dumps(summary))
    return plan, summary


if __name__ == "__main__":
    main()
