"""Op manifests and the sharding-spec algebra used to cost resharding between ops.

A tensor's placement over the GPUs of a stage is `{"R": replicas, "V": partial-sum copies,
"dims": [d0, d1, d2]}` (how many ways each of the three logical dims -- sequence, batch, hidden --
is split); R * V * prod(dims) is the stage size. Each op states the spec it needs for its input
and the spec it produces, depending on its `algo` (0 = column-then-row Megatron sharding, 1 = the
swapped choice). Reference: eth/searching/model_ops.py:10-43 manifests, :90-112 op classes,
:114-169 specs.
"""
from __future__ import annotations

from typing import Dict, List, Optional

from ..contract.config import FIRST_OP, LAYER_OPS, LEGACY_LAYER_OPS, TAIL_OPS

PUBLIC_LAYER_OPS = LAYER_OPS
TP_TUNABLE_OPS = ("enc-attention-qkv", "enc-attention-dense", "enc-MLP-GEMM-1", "enc-MLP-GEMM-2")
NEVER_RECOMPUTE_OPS = (FIRST_OP, "enc-1st-layernorm") + TAIL_OPS


def full_op_list(num_layers: int, legacy: bool = False) -> List[str]:
    layer = LEGACY_LAYER_OPS if legacy else PUBLIC_LAYER_OPS
    return [FIRST_OP] + list(layer) * num_layers + list(TAIL_OPS)


def _spec(r, v, dims) -> Dict[str, object]:
    return {"R": r, "V": v, "dims": list(dims)}


def get_op_spec(op_name: str, tp: int, dp: int, algo: int, input_spec: bool) -> Optional[Dict[str, object]]:
    replicated = _spec(tp, 1, [1, dp, 1])
    hidden_split = _spec(1, 1, [1, dp, tp])
    heads_split = _spec(1, 1, [dp, tp, 1])
    if op_name == FIRST_OP:
        return None if input_spec else replicated
    if op_name in ("enc-1st-layernorm", "enc-2nd-layernorm", "enc-post-attention-dropout", "enc-post-MLP-dropout"):
        return replicated
    if op_name == "final-layernorm":
        return replicated if input_spec else _spec(tp, 1, [dp, 1, 1])
    if op_name in ("enc-attention-qkv", "enc-MLP-GEMM-1"):
        column = algo == 0
        return (replicated if column else hidden_split) if input_spec else (hidden_split if column else replicated)
    if op_name in ("enc-attention-dense", "enc-MLP-GEMM-2"):
        row = algo == 0
        return (hidden_split if row else replicated) if input_spec else (replicated if row else hidden_split)
    if op_name in ("enc-flash-attention", "enc-MLP-gelu"):
        return hidden_split
    if op_name == "enc-attention-score":
        return hidden_split if input_spec else heads_split
    if op_name in ("enc-attention-softmax", "enc-attention-dropout"):
        return heads_split
    if op_name == "enc-attention-context":
        return heads_split if input_spec else hidden_split
    if op_name == "gpt-post-process":
        return _spec(tp, 1, [dp, 1, 1]) if input_spec else None
    raise KeyError(f"unknown op {op_name!r}")
