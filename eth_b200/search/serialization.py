"""Search results on disk: the legacy single-pipeline JSON of the reference
(eth/searching/serialization.py:20-79 -- node_info, model_name, model_size, num_layers, seq_length,
max_position_embeddings, num_attention_heads, hidden_size, global_batch_size, micro_batch_size,
num_stages, num_gpus[], checkpoint_activations[], resharding_stages[], num_ops_in_each_stage[],
model_parallel_size_of_each_op[][], data_parallel_size_of_each_op[][], recompute_ops[][],
algo_of_each_op[][]) and the hybrid `pipe[]` form (:82-151) that normalizes directly."""
from __future__ import annotations

import json

from ..contract.config import LAYER_OPS

OPS_PER_LAYER = len(LAYER_OPS)


def stage_op_counts(layers, ):
    ops = [n * OPS_PER_LAYER for n in layers]
    ops[0] += 1
    ops[-1] += 2
    return ops


def recompute_bitmap(stage_index, num_stages, layers, recompute_layers):
    """Per-op 0/1 list of a stage: the first `recompute_layers` layers are recomputed; embedding
    and the two tail ops never are (reference: never-recompute ops, model_ops.py:102-112)."""
    bits = []
    if stage_index == 0:
        bits.append(0)
    for l in range(layers):
        bits += [1 if l < recompute_layers else 0] * OPS_PER_LAYER
    if stage_index == num_stages - 1:
        bits += [0, 0]
    return bits


def pipeline_to_pipe_dict(p, global_batch, num_layers):
    S = len(p.stages)
    if getattr(p, "op_counts", None):
        # op-granular result of the local search: cuts may fall inside a layer, recompute is per op
        ops = list(p.op_counts)
        rec = [list(m) if m else [0] * n for m, n in zip(p.recompute_masks or [()] * S, ops)]
    else:
        ops = stage_op_counts(p.layers)
        rec = [recompute_bitmap(i, S, p.layers[i], p.recompute_layers[i]) for i in range(S)]
    return {
        "global_batch_size": int(global_batch), "micro_batch_size": int(p.mbs), "num_stages": S,
        "num_gpus": [s.gpus for s in p.stages],
        "checkpoint_activations": [max(r) > 0 for r in rec],
        # a stage in the swapped sharding converts placements at its GEMMs' inputs and outputs
        "resharding_stages": [bool(getattr(s, "algo", 0)) for s in p.stages],
        "num_ops_in_each_stage": ops,
        "model_parallel_size_of_each_op": [[s.tp] * n for s, n in zip(p.stages, ops)],
        "data_parallel_size_of_each_op": [[s.dp] * n for s, n in zip(p.stages, ops)],
        "algo_of_each_op": [[int(getattr(s, "algo", 0))] * n for s, n in zip(p.stages, ops)],
        "recompute_ops": rec,
    }


def dump_pipeline_legacy(p, global_batch, path, args):
    d = pipeline_to_pipe_dict(p, global_batch, args.num_layers)
    out = {"node_info": args.node_info, "model_name": "gpt", "model_size": args.model_size,
           "num_layers": args.num_layers, "seq_length": args.seq_length, "max_position_embeddings": args.seq_length,
           "num_attention_heads": args.num_attention_heads, "hidden_size": args.hidden_size}
    out.update(d)
    with open(path, "w") as f:
        json.dump(out, f, indent=4)
    return out


def dump_hybrid_config(config, path):
    with open(path, "w") as f:
        json.dump(config, f, indent=4)


def load_initial_plan(path, num_layers, gpu_types):
    """A legacy single-pipeline JSON (this module's `dump_pipeline_legacy`, or the reference's) as a
    starting point of the local search; None if it does not describe this model."""
    from .state import PipelinePlan, StagePlan, total_ops
    try:
        with open(path) as f:
            d = json.load(f)
    except (OSError, ValueError):
        return None
    counts = d.get("num_ops_in_each_stage")
    if not counts or sum(counts) != total_ops(num_layers):
        return None
    stages, cursor, gpu_cursor = [], 0, 0
    for i, n in enumerate(counts):
        gpus = d["num_gpus"][i]
        types = tuple(sorted(set(gpu_types[gpu_cursor:gpu_cursor + gpus]))) or (gpu_types[0],)
        stages.append(StagePlan(cursor, cursor + n, gpus, d["model_parallel_size_of_each_op"][i][0],
                                d["data_parallel_size_of_each_op"][i][0], types,
                                algo=int((d.get("algo_of_each_op") or [[0]] * len(counts))[i][0])))
        cursor += n
        gpu_cursor += gpus
    return PipelinePlan(tuple(stages), int(d["micro_batch_size"]))
