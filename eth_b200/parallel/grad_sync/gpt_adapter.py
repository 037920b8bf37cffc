"""GPT op -> logical parameter mapping and per-rank gradient descriptors.

Every parameter of the GPT op graph has a topology-independent logical id
(`gpt.layers.<i>.attention.query_key_value.weight`, ..., `gpt.word_embeddings.weight`) with fixed
sharding semantics: column-parallel weights and biases are cut along dim 0, row-parallel weights
along dim 1, LayerNorm parameters / row-parallel biases / position embeddings are identical
duplicates on every TP rank (reference: eth/runtime/megatron/grad_sync/gpt_adapter.py:19-91;
validation of shapes and of the stage's op range :107-349).
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from .descriptors import LocalGradientBinding, SerializableGradientDescriptor


def _dtype_name(dt) -> str:
    s = str(dt)
    return s[6:] if s.startswith("torch.") else s


def collect_gpt_gradient_metadata(stage, pstate, normalized_config) -> Tuple[List, List]:
    """Descriptors (serialisable) and bindings (local tensors) of all parameters of `stage`."""
    manifest = normalized_config["manifest"]
    begin, end = pstate.op_range
    want_ranges = [tuple(r) for r in getattr(pstate, "chunk_ranges", [(begin, end)])]
    have_ranges = [tuple(r) for r in getattr(stage, "chunk_ranges", [(stage.op_begin, stage.op_end)])]
    if have_ranges != want_ranges:
        raise ValueError(f"stage owns ops {have_ranges} but the topology says {want_ranges}")
    for op in stage.ops:
        want = manifest["ordered_ops"][op.op_index]["name"]
        if op.name != want:
            raise ValueError(f"op {op.op_index} is {op.name!r} but the manifest says {want!r}")
    descriptors, bindings = [], []
    seen = set()

    def chunk_of(op_index: int) -> int:
        return next(c for c, (lo, hi) in enumerate(have_ranges) if lo <= op_index < hi)
    tp, tp_rank = pstate.tp_size, pstate.tp_rank
    for e in stage.unique_entries():
        spec, p = e.spec, e.param
        if spec.logical_id in seen:
            raise ValueError(f"duplicate logical parameter {spec.logical_id} in one stage")
        seen.add(spec.logical_id)
        sharded = spec.partition_dim >= 0
        expect = spec.local_shape(tp)
        if tuple(p.shape) != tuple(expect):
            raise ValueError(f"{spec.logical_id}: local shape {tuple(p.shape)} != expected {tuple(expect)}")
        if sharded and spec.full_shape[spec.partition_dim] % (tp * spec.partition_stride):
            raise ValueError(f"{spec.logical_id}: axis not divisible by TP {tp}")
        order_key = _order_key(spec.logical_id)
        descriptors.append(SerializableGradientDescriptor(
            logical_param_id=spec.logical_id, shared_weight_id=None, shared_weight_root=False,
            logical_region_key=spec.logical_id, semantic_order_key=order_key, global_rank=pstate.rank,
            model_impl=normalized_config["model_impl"], op_manifest_hash=manifest["hash"],
            pipeline_id=pstate.pipeline_id, stage_id=pstate.stage_id, model_chunk_id=chunk_of(e.op.op_index),
            global_op_index=e.op.op_index, manifest_op_name=e.op.name, runtime_op_name=type(e.op).__name__,
            relative_parameter_name=spec.local_name, stage_global_op_begin=begin, stage_global_op_end=end,
            local_tp_degree=tp, local_tp_rank=tp_rank, local_dp_degree=pstate.dp_size, local_dp_rank=pstate.dp_rank,
            local_cp_degree=1, local_cp_rank=0, stage_ranks=tuple(pstate.stage.stage_ranks),
            local_tp_group_ranks=tuple(pstate.tp_group_ranks), local_dp_group_ranks=tuple(pstate.dp_group_ranks),
            full_shape=tuple(spec.full_shape), local_shape=tuple(p.shape), tensor_parallel=sharded,
            tp_replica_semantics=None if sharded else "identical_duplicate",
            partition_dim=spec.partition_dim, partition_stride=spec.partition_stride,
            parameter_dtype=_dtype_name(p.dtype), gradient_dtype=_dtype_name(p.main_grad.dtype),
            requires_grad=True))
        bindings.append(LocalGradientBinding(spec.logical_id, p, p.main_grad, p.main_grad.device))
    return descriptors, bindings


def _order_key(logical_id: str) -> tuple:
    """Model order: embeddings, layers by index, final LayerNorm; then the name."""
    parts = logical_id.split(".")
    if len(parts) > 2 and parts[1] == "layers":
        return (1, int(parts[2]), ".".join(parts[3:]))
    if "embeddings" in logical_id:
        return (0, 0, logical_id)
    return (2, 0, logical_id)
