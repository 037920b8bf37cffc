"""Op profiler: times every op of the one-layer GPT op list at a given tensor-parallel degree.

    torchrun --nproc-per-node <tp> -m eth_b200.profiler.op_profiler --prof-tp-size <tp> \
        --prof-path out/ --prof-model-size 1_3B [--prof-mbs-list 1 2 4 8]

For every micro-batch size and op: build the op alone (the real stage-program op with its real
kernels, including the fused tensor-parallel reductions), feed random boundary tensors of the right
shapes, and time forward and backward separately with CUDA events on the launching stream (the
reference brackets host wall-clock with device synchronisation, eth/profiler/op_profiler.py:326-358).
Output: `gpt_<size>_mbs<m>_tp<t>_algo<a>.csv` with header
`op_name, forward-compute, backward-compute, input_size, output_size, weights, activations,
fwd_reserved, bwd_reserved` (times in microseconds, sizes in MB; :424-445) and a pickle cache.
The algo-1 file is measured with the four tensor-parallel GEMM ops in their swapped sharding
(placement conversions at their inputs and outputs included); every other op has one form, so
its measurement is shared by both files through the cache key (`op_key`; reference :221-228). A
failed op is recorded with the reference's sentinel 1e7 (:528-530).

With `--prof-num-nodes N --prof-node-rank r` the micro-batch sizes are dealt out to the nodes by
estimated cost (tokens per micro-batch), largest first onto the least loaded node, so that N nodes
of the same GPU type profile disjoint shares (reference :452-487 splits by a previous run's times).
"""
from __future__ import annotations

import csv
import os
import pickle
import sys

import torch
import torch.distributed as dist

from ..contract.config import manifest_size
from ..models.gpt_ops import LIVE_AFTER, GPTModelConfig, TPComm
from ..models.stage import GPTStage, MicroBatch
from ..search.profile_db import OP_HEADER
from .model_configs import gpt_profile_shape

FAILED = 1.0e7
MB = 1024.0 * 1024.0


def _tensor_mb(t) -> float:
    return t.numel() * t.element_size() / MB if isinstance(t, torch.Tensor) else 0.0


def _ctx_mb(ctx) -> float:
    seen, total = set(), 0.0
    for v in ctx.values():
        if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
            seen.add(v.data_ptr())
            total += _tensor_mb(v)
    return total


def profile_op(stage: GPTStage, mbs: int, seq: int, vocab: int, warmup: int, repeat: int, device):
    """Returns the CSV row values of the single op held by `stage`."""
    op = stage.ops[0]
    cfg = stage.cfg
    tokens = mbs * seq
    prev = stage.descriptors[stage.op_begin - 1]["name"] if stage.op_begin > 0 else None
    in_shapes = stage.boundary_shapes(LIVE_AFTER[prev], tokens) if prev else {}
    out_shapes = stage.boundary_shapes(stage.output_spec, tokens)
    dt = cfg.params_dtype

    def make_inputs():
        env = {n: torch.randn(s, device=device, dtype=dt) * 0.1 for n, s in in_shapes.items()}
        if op.name == "encoder-embedding":
            env["enc_input_ids"] = torch.randint(0, vocab, (mbs, seq), device=device)
        if op.name == "gpt-post-process":
            env["labels"] = torch.randint(0, vocab, (mbs, seq), device=device)
        if "output_bias" in env:
            env["output_bias"] = torch.zeros(in_shapes["output_bias"], device=device, dtype=dt)
        return env

    def make_grads():
        g = {}
        for n, s in out_shapes.items():
            g[n] = torch.randn(s, device=device, dtype=torch.float32 if n == "output_bias" else dt) * 0.1
        if op.name == "gpt-post-process":
            g = {"output": torch.ones(tokens, device=device) / tokens}
        return g

    mb = MicroBatch(index=0, batch=mbs, seq=seq, global_step=0, dp_rank=0)
    fwd_ms = bwd_ms = 0.0
    act_mb = in_mb = out_mb = fwd_res = bwd_res = 0.0
    for it in range(warmup + repeat):
        env, ctx = make_inputs(), {}
        mb.ctxs = {op.op_index: ctx}
        in_mb = sum(_tensor_mb(v) for k, v in env.items() if k in in_shapes or k == "enc_input_ids")
        torch.cuda.synchronize()
        base = torch.cuda.memory_allocated()
        torch.cuda.reset_peak_memory_stats()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        op.fwd(env, ctx, mb)
        e1.record()
        outs = {k: v for k, v in env.items() if k in out_shapes or k == "output"}
        grads = make_grads()
        torch.cuda.synchronize()
        fwd_res = (torch.cuda.max_memory_allocated() - base) / MB
        torch.cuda.reset_peak_memory_stats()
        base2 = torch.cuda.memory_allocated()
        e1b = torch.cuda.Event(enable_timing=True)
        e1b.record()
        op.bwd(grads, ctx, mb)
        e2.record()
        e2.synchronize()
        bwd_res = (torch.cuda.max_memory_allocated() - base2) / MB
        if it >= warmup:
            fwd_ms += e0.elapsed_time(e1)
            bwd_ms += e1b.elapsed_time(e2)
        act_mb = _ctx_mb(ctx)
        out_mb = sum(_tensor_mb(v) for v in outs.values())
    weights_mb = sum(e.numel * e.param.element_size() for e in stage.unique_entries()) / MB
    return [op.name, fwd_ms / repeat * 1e3, bwd_ms / repeat * 1e3, in_mb, out_mb, weights_mb, act_mb,
            max(fwd_res, 0.0), max(bwd_res, 0.0)]


ALGO_OPS = ("enc-attention-qkv", "enc-attention-dense", "enc-MLP-GEMM-1", "enc-MLP-GEMM-2")


def op_key(model_size: str, mbs: int, tp_size: int, op_name: str, op_index: int, algo: int):
    """Cache key of one measurement: ops without a second sharding choice share it across algos."""
    return (model_size, mbs, tp_size, op_index, op_name, algo if op_name in ALGO_OPS and tp_size > 1 else 0)


def node_share(mbs_list, num_nodes: int, node_rank: int):
    """The micro-batch sizes this node profiles: longest first onto the least loaded node."""
    if num_nodes <= 1:
        return list(mbs_list)
    load, mine = [0] * num_nodes, []
    for mbs in sorted(mbs_list, reverse=True):
        node = load.index(min(load))
        load[node] += mbs
        if node == node_rank:
            mine.append(mbs)
    return sorted(mine)


def run_profile(args, tp_size: int, tp_rank: int, group, device):
    shape = gpt_profile_shape(args.prof_model_size)
    mbs_list = node_share(args.prof_mbs_list or [1, 2, 4, 8], getattr(args, "prof_num_nodes", 1) or 1,
                          getattr(args, "prof_node_rank", 0) or 0)
    n_ops = manifest_size(1)
    cache_path = args.prof_cache_file
    cache = {}
    if cache_path and os.path.exists(cache_path):
        with open(cache_path, "rb") as f:
            cache = pickle.load(f)
    multiple = 128 * tp_size
    padded_vocab = (shape["vocab"] + multiple - 1) // multiple * multiple
    cfg = GPTModelConfig(num_layers=1, hidden_size=shape["hidden_size"], num_attention_heads=shape["num_attention_heads"],
                         seq_length=shape["seq_length"], max_position_embeddings=shape["seq_length"],
                         padded_vocab_size=padded_vocab, hidden_dropout=0.1, params_dtype=torch.bfloat16,
                         grad_dtype=torch.float32)
    backend = None
    if tp_size > 1:
        try:
            from ..parallel.fused_tp import FusedTPBackend
            backend = FusedTPBackend(tuple(range(tp_size)), tp_rank, group, device, max(mbs_list) * shape["seq_length"],
                                     shape["hidden_size"], torch.bfloat16)
        except Exception as exc:  # fall back to NCCL reductions
            print(f"[op_profiler] fused TP backend unavailable: {exc}", file=sys.stderr)
    tp = TPComm(tp_size, tp_rank, group, backend)
    warmup, repeat = args.prof_warmup_times, args.prof_repeat_times[0]
    names = [d["name"] for d in GPTStage(cfg, 0, 1, tp=TPComm(), device="cpu").descriptors]
    for mbs, algo in ((m, a) for m in mbs_list for a in (0, 1)):
        rows = []
        for i in range(n_ops):
            key = op_key(args.prof_model_size, mbs, tp_size, names[i], i, algo)
            if key in cache:
                rows.append(cache[key])
                continue
            try:
                stage = GPTStage(cfg, i, i + 1, tp=tp, device=device, fuse=False, algo_ops=[algo])
                row = profile_op(stage, mbs, shape["seq_length"], shape["vocab"], warmup, repeat, device)
                del stage
            except Exception as exc:
                print(f"[op_profiler] op {i} mbs {mbs} failed: {exc}", file=sys.stderr)
                row = [f"op{i}", FAILED, FAILED, 0, 0, 0, 0, 0, 0]
            if tp_size > 1:
                # all ranks report the slowest rank's time
                t = torch.tensor(row[1:3], device=device, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                row[1:3] = t.tolist()
            cache[key] = row
            rows.append(row)
            torch.cuda.empty_cache()
        if tp_rank == 0:
            path = os.path.join(args.prof_path, f"gpt_{args.prof_model_size}_mbs{mbs}_tp{tp_size}_algo{algo}.csv")
            with open(path, "w", newline="") as f:
                w = csv.writer(f)
                w.writerow(OP_HEADER)
                for r in rows:
                    w.writerow([r[0]] + [f"{x:.3f}" for x in r[1:3]] + [f"{x:.4f}" for x in r[3:]])
    if tp_rank == 0 and cache_path:
        with open(cache_path, "wb") as f:
            pickle.dump(cache, f)


def main(argv=None):
    from ..runtime.arguments import build_parser
    args = build_parser().parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    tp = args.prof_tp_size or world
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    os.makedirs(args.prof_path, exist_ok=True)
    run_profile(args, tp, rank % tp, None, device)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
