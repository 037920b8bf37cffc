"""The `gpt_config.json` contract: canonical form of a heterogeneous-pipeline (HPP) GPT config.

Same public schema as the reference normalizer (eth/runtime/megatron/config_normalization.py):
allowed top-level keys (:38-55) and per-pipeline keys (:57-77); the 3 + 10*L op manifest with a
sha256 hash (:91-136); every topology field accepted per stage (`*_of_each_stage`) or per op
(`*_of_each_op`), constant inside a stage (:209-246); TP in {1,2,4,6,8}, CP == 1,
num_gpus == TP*DP*CP, batch divisibility, hidden/heads divisible by TP (:272-311, 372-386); and the
derived `world_size`, `total_gbs`, `pipeline_sample_offsets`, `topology_fingerprint`, `config_hash`
(:387-432). Hashes are sha256 over compact sorted-key JSON, so a config normalized here and by the
reference carries the same `config_hash`.

The implementation is a small declarative validator (`_Field` specs + dataclass-free dict output)
rather than a port: the output is plain JSON-serialisable dicts because that *is* the contract.
"""
from __future__ import annotations

import ast
import copy
import hashlib
import json
import warnings
from types import SimpleNamespace
from typing import Any, Dict, List, Optional, Sequence

LAYER_OPS = (
    "enc-1st-layernorm",
    "enc-attention-qkv",
    "enc-flash-attention",
    "enc-attention-dense",
    "enc-post-attention-dropout",
    "enc-2nd-layernorm",
    "enc-MLP-GEMM-1",
    "enc-MLP-gelu",
    "enc-MLP-GEMM-2",
    "enc-post-MLP-dropout",
)
FIRST_OP = "encoder-embedding"
TAIL_OPS = ("final-layernorm", "gpt-post-process")
MODEL_IMPLS = {"gpt": {"id": "gpt", "ops_per_layer": len(LAYER_OPS), "layer_schema": LAYER_OPS}}

SUPPORTED_TP = (1, 2, 4, 6, 8)

TOP_LEVEL_KEYS = frozenset({
    "config_hash", "hidden_size", "manifest", "max_position_embeddings", "model_impl", "model_name",
    "model_size", "node_info", "num_attention_heads", "num_layers", "pipe",
    "pipeline_sample_offsets", "seq_length", "topology_fingerprint", "total_gbs", "world_size",
})
PIPE_KEYS = frozenset({
    "algo_of_each_op", "algo_of_each_stage", "checkpoint_activations",
    "context_parallel_size_of_each_op", "context_parallel_size_of_each_stage",
    "data_parallel_size_of_each_op", "data_parallel_size_of_each_stage", "global_batch_size",
    "micro_batch_size", "model_impl", "model_parallel_size_of_each_op",
    "model_parallel_size_of_each_stage", "node_info", "num_gpus", "num_ops_in_each_stage",
    "num_stages", "pipeline_index", "recompute_ops", "resharding_stages",
})
# (field stem, default when both spellings are absent -- only CP has one)
TOPOLOGY_STEMS = ("model_parallel_size", "data_parallel_size", "context_parallel_size", "algo")


class ConfigError(ValueError):
    """Raised for any violation of the config contract."""


def canonical_hash(value: Any) -> str:
    blob = json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=True)
    return hashlib.sha256(blob.encode("utf-8")).hexdigest()


def manifest_size(num_layers: int, model_impl: str = "gpt") -> int:
    return 3 + num_layers * MODEL_IMPLS[model_impl]["ops_per_layer"]


def build_manifest(model_impl: str, num_layers: int) -> Dict[str, Any]:
    """Ordered op list `[embedding] + layer ops * L + [final-layernorm, gpt-post-process]`."""
    if model_impl not in MODEL_IMPLS:
        raise ConfigError(
            f"unsupported model_impl {model_impl!r}; expected one of {', '.join(sorted(MODEL_IMPLS))}")
    spec = MODEL_IMPLS[model_impl]
    names: List[tuple] = [(FIRST_OP, None)]
    for layer in range(num_layers):
        names.extend((op, layer) for op in spec["layer_schema"])
    names.extend((op, None) for op in TAIL_OPS)
    ordered = [{"op_index": i, "name": n, "layer_index": layer} for i, (n, layer) in enumerate(names)]
    manifest = {"id": spec["id"], "ops_per_layer": spec["ops_per_layer"], "ordered_ops": ordered}
    manifest["hash"] = canonical_hash(manifest)
    return manifest


def validate_runtime_manifest(runtime_ops: Sequence[Dict[str, Any]], manifest: Dict[str, Any]) -> None:
    """The model's own op list must be exactly the manifest (names and indices, in order)."""
    want = manifest["ordered_ops"]
    if len(runtime_ops) != len(want):
        raise ConfigError(
            f"runtime GPT manifest mismatch: expected {len(want)} ops, got {len(runtime_ops)}")
    for pos, (have, exp) in enumerate(zip(runtime_ops, want)):
        got = (have.get("op_index"), have.get("name"))
        need = (exp["op_index"], exp["name"])
        if got != need:
            raise ConfigError(f"runtime GPT manifest mismatch at op {pos}: expected {need}, got {got}")


def _is_pos_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v > 0


def _resolve_model_impl(config: Dict[str, Any], op_totals: Sequence[int]) -> str:
    layers = config.get("num_layers")
    if not _is_pos_int(layers):
        raise ConfigError("num_layers must be a positive integer")
    top = config.get("model_impl")
    per_pipe = {p.get("model_impl") for p in config["pipe"] if p.get("model_impl")}
    if len(per_pipe) > 1:
        raise ConfigError("different manifests requested by per-pipeline model_impl values")
    if per_pipe and top and top not in per_pipe:
        raise ConfigError("top-level model_impl conflicts with per-pipeline model_impl")
    if per_pipe:
        top = next(iter(per_pipe))
    guesses = []
    for total in op_totals:
        fits = [name for name in MODEL_IMPLS if total == manifest_size(layers, name)]
        if len(fits) != 1:
            raise ConfigError(f"manifest size {total} does not uniquely match a supported model_impl")
        guesses.append(fits[0])
    if len(set(guesses)) != 1:
        raise ConfigError("different manifests inferred across pipelines")
    if top is not None:
        build_manifest(top, layers)  # validates the name
        if top != guesses[0]:
            raise ConfigError(f"model_impl {top!r} conflicts with pipeline manifest size")
        return top
    warnings.warn(f"model_impl inferred as {guesses[0]}; regenerate the config with an explicit value",
                  UserWarning, stacklevel=3)
    return guesses[0]


def _stage_list(pipe, key, stages):
    v = pipe.get(key)
    if not isinstance(v, list) or len(v) != stages:
        raise ConfigError(f"{key} stage list length must equal num_stages")
    return v


def _per_op_field(pipe, stem, stage_ops):
    """Canonical per-op nested list of one topology field from either spelling."""
    k_stage, k_op = f"{stem}_of_each_stage", f"{stem}_of_each_op"
    by_stage, by_op = pipe.get(k_stage), pipe.get(k_op)
    if by_stage is None and by_op is None and stem == "context_parallel_size":
        by_stage = [1] * len(stage_ops)
    from_stage = None
    if by_stage is not None:
        if not isinstance(by_stage, list) or len(by_stage) != len(stage_ops):
            raise ConfigError(f"{k_stage} stage list length must equal num_stages")
        from_stage = [[v] * n for v, n in zip(by_stage, stage_ops)]
    if by_op is not None:
        if not isinstance(by_op, list) or len(by_op) != len(stage_ops):
            raise ConfigError(f"{k_op} stage list length must equal num_stages")
        out = []
        for s, (vals, n) in enumerate(zip(by_op, stage_ops)):
            if not isinstance(vals, list) or len(vals) != n:
                raise ConfigError(f"{k_op} stage {s} length must equal its op count")
            if len(set(vals)) != 1:
                raise ConfigError(f"intra-stage constancy violated for {k_op} at stage {s}")
            out.append(list(vals))
        if from_stage is not None and out != from_stage:
            raise ConfigError(f"brief and expanded {stem} values conflict")
        return out
    if from_stage is None:
        raise ConfigError(f"missing {k_stage} or {k_op}")
    return from_stage


def _normalize_pipeline(src: Dict[str, Any], index: int, n_ops: int) -> Dict[str, Any]:
    pipe = copy.deepcopy(src)
    stages = pipe.get("num_stages")
    if not _is_pos_int(stages):
        raise ConfigError(f"pipeline {index} num_stages must be positive")
    stage_ops = _stage_list(pipe, "num_ops_in_each_stage", stages)
    if not all(_is_pos_int(c) for c in stage_ops):
        raise ConfigError("num_ops_in_each_stage values must be positive integers")
    if sum(stage_ops) != n_ops:
        raise ConfigError(
            f"manifest size mismatch in pipeline {index}: expected {n_ops}, got {sum(stage_ops)}")
    fields = {f"{stem}_of_each_op": _per_op_field(pipe, stem, stage_ops) for stem in TOPOLOGY_STEMS}
    tp = [v[0] for v in fields["model_parallel_size_of_each_op"]]
    dp = [v[0] for v in fields["data_parallel_size_of_each_op"]]
    cp = [v[0] for v in fields["context_parallel_size_of_each_op"]]
    for s, c in enumerate(cp):
        if c != 1:
            raise ConfigError(f"context parallel stage {s} must be 1 for block-wise sync")
    for label, vals in (("TP", tp), ("DP", dp), ("CP", cp)):
        if not all(_is_pos_int(v) for v in vals):
            raise ConfigError(f"{label} values must be positive integers")
    for s, t in enumerate(tp):
        if t not in SUPPORTED_TP:
            raise ConfigError(
                f"unsupported TP value {t} in pipeline {index} stage {s}; supported TP values are "
                + ", ".join(map(str, SUPPORTED_TP)))
    gpus = _stage_list(pipe, "num_gpus", stages)
    for s, (g, t, d, c) in enumerate(zip(gpus, tp, dp, cp)):
        if g != t * d * c:
            raise ConfigError(
                f"stage product mismatch in pipeline {index} stage {s}: num_gpus={g}, TP*DP*CP={t * d * c}")
    mbs, gbs = pipe.get("micro_batch_size"), pipe.get("global_batch_size")
    if not _is_pos_int(mbs):
        raise ConfigError("micro_batch_size must be a positive integer")
    if not _is_pos_int(gbs):
        raise ConfigError("global_batch_size must be a positive integer")
    if gbs % mbs:
        raise ConfigError("micro batch divisibility requires GBS % micro_batch_size == 0")
    for s, d in enumerate(dp):
        if mbs % d:
            raise ConfigError(
                f"micro batch divisibility failed for pipeline {index} stage {s}: micro_batch_size % DP != 0")
    recompute = _stage_list(pipe, "recompute_ops", stages)
    for s, (vals, n) in enumerate(zip(recompute, stage_ops)):
        if not isinstance(vals, list) or len(vals) != n:
            raise ConfigError(f"recompute_ops stage {s} length must equal its op count")
    out = {
        "pipeline_index": index,
        "global_batch_size": gbs,
        "micro_batch_size": mbs,
        "num_stages": stages,
        "num_gpus": list(gpus),
        "num_ops_in_each_stage": list(stage_ops),
        "checkpoint_activations": list(_stage_list(pipe, "checkpoint_activations", stages)),
        "resharding_stages": list(_stage_list(pipe, "resharding_stages", stages)),
        "recompute_ops": recompute,
    }
    out.update(fields)
    return out


def normalize_flexpipe_config(config: Dict[str, Any], world_size: Optional[int] = None) -> Dict[str, Any]:
    """Unique canonical representation of an HPP GPT config (raises ConfigError on violations)."""
    if not isinstance(config, dict):
        raise ConfigError("config must be a mapping")
    extra = sorted(set(config) - TOP_LEVEL_KEYS)
    if extra:
        raise ConfigError(f"unknown top-level config field(s): {', '.join(extra)}")
    pipes = config.get("pipe")
    if not isinstance(pipes, list) or not pipes:
        raise ConfigError("config must contain at least one pipeline")
    totals = []
    for i, pipe in enumerate(pipes):
        if not isinstance(pipe, dict):
            raise ConfigError(f"pipeline {i} must be a mapping")
        extra = sorted(set(pipe) - PIPE_KEYS)
        if extra:
            raise ConfigError(f"pipeline {i} has unknown field(s): {', '.join(extra)}")
        counts = pipe.get("num_ops_in_each_stage")
        if not isinstance(counts, list) or not counts:
            raise ConfigError(f"pipeline {i} is missing num_ops_in_each_stage")
        totals.append(sum(counts))
    impl = _resolve_model_impl(config, totals)
    manifest = build_manifest(impl, config["num_layers"])
    norm_pipes = [_normalize_pipeline(p, i, len(manifest["ordered_ops"])) for i, p in enumerate(pipes)]
    hidden, heads = config.get("hidden_size"), config.get("num_attention_heads")
    for pi, pipe in enumerate(norm_pipes):
        for si, vals in enumerate(pipe["model_parallel_size_of_each_op"]):
            t = vals[0]
            if not isinstance(hidden, int) or hidden % t or not isinstance(heads, int) or heads % t:
                raise ConfigError(
                    f"TP constraint failed in pipeline {pi} stage {si}: hidden_size={hidden}, "
                    f"num_attention_heads={heads}, TP={t}")
    world = sum(sum(p["num_gpus"]) for p in norm_pipes)
    if world_size is not None and world_size != world:
        raise ConfigError(f"world size mismatch: expected {world}, got {world_size}")
    offsets, running = [], 0
    for p in norm_pipes:
        offsets.append(running)
        running += p["global_batch_size"]
    out = {k: copy.deepcopy(v) for k, v in config.items() if k not in ("pipe", "model_impl")}
    out.update({
        "model_impl": impl,
        "manifest": manifest,
        "pipe": norm_pipes,
        "world_size": world,
        "total_gbs": running,
        "pipeline_sample_offsets": offsets,
    })
    topo_keys = ("num_gpus", "num_ops_in_each_stage", "model_parallel_size_of_each_op",
                 "data_parallel_size_of_each_op", "context_parallel_size_of_each_op")
    out["topology_fingerprint"] = canonical_hash(
        {"world_size": world, "pipelines": [{k: p[k] for k in topo_keys} for p in norm_pipes]})
    out["config_hash"] = canonical_hash(out)
    return out


def load_config(path: str, world_size: Optional[int] = None) -> Dict[str, Any]:
    with open(path) as f:
        return normalize_flexpipe_config(json.load(f), world_size)


# ------------------------------------------------------------------------------------------
# runtime view of a normalized config
# ------------------------------------------------------------------------------------------
def parse_mbs_sequence(value):
    if isinstance(value, str):
        try:
            value = ast.literal_eval(value)
        except (SyntaxError, ValueError) as exc:
            raise ConfigError("mbs_seq must be a literal list") from exc
    if value is None:
        return []
    if not isinstance(value, list):
        raise ConfigError("mbs_seq must be a list")
    return value


_PER_PIPE_ATTRS = {
    "num_gpus_each_pipe": "num_gpus",
    "num_ops_in_each_stage_each_pipe": "num_ops_in_each_stage",
    "micro_batch_size_each_pipe": "micro_batch_size",
    "num_stages_each_pipe": "num_stages",
    "algo_of_each_op_each_pipe": "algo_of_each_op",
    "model_parallel_size_of_each_op_each_pipe": "model_parallel_size_of_each_op",
    "data_parallel_size_of_each_op_each_pipe": "data_parallel_size_of_each_op",
    "context_parallel_size_of_each_op_each_pipe": "context_parallel_size_of_each_op",
    "recompute_ops_each_pipe": "recompute_ops",
    "resharding_stages_each_pipe": "resharding_stages",
    "checkpoint_activations_each_pipe": "checkpoint_activations",
    "global_batch_size_each_pipe": "global_batch_size",
}
_LOCAL_ATTRS = ("global_batch_size", "micro_batch_size", "num_gpus", "num_ops_in_each_stage",
                "num_stages", "algo_of_each_op", "model_parallel_size_of_each_op",
                "data_parallel_size_of_each_op", "context_parallel_size_of_each_op",
                "recompute_ops", "resharding_stages", "checkpoint_activations")


def apply_normalized_config_to_args(args, normalized):
    """Fill the runtime argument namespace from a canonical config: rank -> (pipeline, stage,
    rank offset) maps with ranks laid out pipeline-major then stage-major, per-pipeline lists,
    this rank's pipeline fields, the per-pipeline micro-batch schedule `mbs_seq`
    (`[[mbs, seq_len], ...]`) and `nominal_global_loss_scale = sum(mbs * seq_len)`
    (reference: config_normalization.py:448-546)."""
    if args.world_size != normalized["world_size"]:
        raise ConfigError(f"world size mismatch: expected {normalized['world_size']}, got {args.world_size}")
    if not 0 <= args.rank < args.world_size:
        raise ConfigError(f"rank {args.rank} is outside world size {args.world_size}")
    for k, v in normalized.items():
        if k != "pipe":
            setattr(args, k, copy.deepcopy(v))
    args.manifest_hash = normalized["manifest"]["hash"]
    args.num_ops_each_layer = normalized["manifest"]["ops_per_layer"]
    pipes = normalized["pipe"]
    args.pipe_num = len(pipes)
    for dst, src in _PER_PIPE_ATTRS.items():
        setattr(args, dst, [copy.deepcopy(p[src]) for p in pipes])
    args.sum_gpus_each_pipe = [sum(p["num_gpus"]) for p in pipes]
    args.rank_to_pipe, args.rank_to_stage, args.rank_to_offset = [], [], []
    args.offset_list_each_pipe = []
    base = 0
    for pi, p in enumerate(pipes):
        args.offset_list_each_pipe.append(base)
        for si, n in enumerate(p["num_gpus"]):
            args.rank_to_pipe += [pi] * n
            args.rank_to_stage += [si] * n
            args.rank_to_offset += [base] * n
        base += sum(p["num_gpus"])
    args.offset_list_each_pipe.append(base)
    args.current_pipe = args.rank_to_pipe[args.rank]
    args.offset = args.rank_to_offset[args.rank]
    mine = pipes[args.current_pipe]
    for k in _LOCAL_ATTRS:
        setattr(args, k, copy.deepcopy(mine[k]))
    args.num_op = sum(args.num_ops_in_each_stage)
    seqs = parse_mbs_sequence(getattr(args, "mbs_seq", []))
    if not seqs:
        seqs = [[[p["micro_batch_size"], normalized["seq_length"]]] * (p["global_batch_size"] // p["micro_batch_size"])
                for p in pipes]
    if len(seqs) != len(pipes):
        raise ConfigError("mbs_seq must contain one sequence per pipeline")
    for pi, (seq, p) in enumerate(zip(seqs, pipes)):
        try:
            total = sum(item[0] for item in seq)
        except (IndexError, TypeError) as exc:
            raise ConfigError(f"mbs_seq pipeline {pi} is malformed") from exc
        if total != p["global_batch_size"]:
            raise ConfigError(f"mbs_seq pipeline {pi} sums to {total}, expected {p['global_batch_size']}")
    args.mbs_seq = seqs
    args.nominal_global_loss_scale = float(sum(m * s for seq in seqs for m, s in seq))
    if args.nominal_global_loss_scale <= 0:
        raise ConfigError("nominal_global_loss_scale must be positive")
    return args


def runtime_view(normalized: Dict[str, Any], rank: int, world_size: Optional[int] = None, mbs_seq=None):
    """Convenience: a fresh namespace populated by `apply_normalized_config_to_args`."""
    ns = SimpleNamespace(rank=rank, world_size=world_size or normalized["world_size"], mbs_seq=mbs_seq or [])
    return apply_normalized_config_to_args(ns, normalized)


# ------------------------------------------------------------------------------------------
# config builders (fixtures and uniform layouts)
# ------------------------------------------------------------------------------------------
def make_pipe(stage_ops, tp, dp, gbs=24, mbs=8, recompute=None, algo=None):
    n = len(stage_ops)
    return {
        "global_batch_size": gbs,
        "micro_batch_size": mbs,
        "num_stages": n,
        "num_gpus": [t * d for t, d in zip(tp, dp)],
        "checkpoint_activations": [False] * n,
        "resharding_stages": [False] * n,
        "num_ops_in_each_stage": list(stage_ops),
        "model_parallel_size_of_each_stage": list(tp),
        "data_parallel_size_of_each_stage": list(dp),
        "context_parallel_size_of_each_stage": [1] * n,
        "algo_of_each_stage": list(algo) if algo is not None else [0] * n,
        "recompute_ops": recompute if recompute is not None else [[0] * c for c in stage_ops],
    }


def make_config(pipes, num_layers=4, hidden_size=64, num_attention_heads=8, seq_length=32,
                model_size="fixture", max_position_embeddings=None):
    return {
        "model_name": "gpt",
        "model_impl": "gpt",
        "model_size": model_size,
        "num_layers": num_layers,
        "seq_length": seq_length,
        "max_position_embeddings": max_position_embeddings or seq_length,
        "num_attention_heads": num_attention_heads,
        "hidden_size": hidden_size,
        "pipe": pipes,
    }


def split_layers_evenly(num_layers: int, num_stages: int) -> List[int]:
    """Op counts per stage for layer-aligned cuts: embedding joins the first stage, the two tail
    ops join the last."""
    base, rem = divmod(num_layers, num_stages)
    layers = [base + (1 if s < rem else 0) for s in range(num_stages)]
    ops = [n * len(LAYER_OPS) for n in layers]
    ops[0] += 1
    ops[-1] += 2
    return ops


def uniform_config(model: Dict[str, Any], pp: int, tp: int, dp: int, gbs: int, mbs: int,
                   num_pipelines: int = 1, stage_layers: Optional[Sequence[int]] = None):
    """A homogeneous layout: `num_pipelines` identical pipelines of `pp` stages, each TP x DP."""
    if stage_layers is not None:
        ops = [n * len(LAYER_OPS) for n in stage_layers]
        ops[0] += 1
        ops[-1] += 2
    else:
        ops = split_layers_evenly(model["num_layers"], pp)
    pipes = [make_pipe(ops, [tp] * pp, [dp] * pp, gbs=gbs // num_pipelines, mbs=mbs)
             for _ in range(num_pipelines)]
    return make_config(pipes, num_layers=model["num_layers"], hidden_size=model["hidden_size"],
                       num_attention_heads=model["num_attention_heads"], seq_length=model["seq_length"],
                       model_size=model.get("model_size", "custom"),
                       max_position_embeddings=model.get("max_position_embeddings"))


GPT_SIZES = {
    # name: (layers, hidden, heads, seq)  -- reference presets: eth/searching/arguments.py:10-18
    "350M": dict(num_layers=24, hidden_size=1024, num_attention_heads=16, seq_length=2048),
    "1_3B": dict(num_layers=24, hidden_size=2048, num_attention_heads=32, seq_length=2048),
    "2_6B": dict(num_layers=32, hidden_size=2560, num_attention_heads=32, seq_length=2048),
    "6_7B": dict(num_layers=32, hidden_size=4096, num_attention_heads=32, seq_length=2048),
    "13B": dict(num_layers=40, hidden_size=5120, num_attention_heads=40, seq_length=2048),
    "70B": dict(num_layers=80, hidden_size=8192, num_attention_heads=64, seq_length=2048),
}


def heterogeneous_config_fixtures():
    """The tracked minimum topology sweep (same layouts as config_normalization.py:549-612)."""
    P, C = make_pipe, make_config
    return [
        C([P([43], [1], [1]), P([11, 32], [1, 1], [1, 2])]),
        C([P([21, 22], [1, 2], [1, 1]), P([11, 32], [1, 1], [2, 1])]),
        C([P([11, 32], [2, 1], [1, 1]), P([21, 22], [1, 1], [1, 2])]),
        C([P([43], [1], [2], gbs=8), P([43], [2], [1], gbs=16), P([43], [1], [2], gbs=24)]),
        C([P([11, 20, 12], [1, 2, 1], [1, 1, 1]), P([21, 10, 12], [1, 1, 1], [2, 1, 1])]),
        C([P([10, 33], [1, 2], [2, 1]), P([30, 13], [2, 1], [1, 2])]),
    ]


def gpt_e2e_fixtures():
    """Named launcher fixtures (config_normalization.py:615-654)."""
    P, C = make_pipe, make_config
    return {
        "canonical-4r-equal-gbs": C([P([43], [1], [2]), P([43], [2], [1])]),
        "reference-1r-canonical4-global-batch": C([P([43], [1], [1], gbs=48)]),
        "brief-6r-equal-gbs": C([P([21, 22], [1, 2], [1, 1]), P([11, 32], [1, 1], [2, 1])]),
        "hetero-6r-swapped-stages": C([P([11, 32], [2, 1], [1, 1]), P([21, 22], [1, 1], [1, 2])]),
        "canonical-6r-three-pipeline": C([P([43], [1], [2], gbs=12, mbs=4), P([43], [2], [1], gbs=16, mbs=4),
                                          P([43], [1], [2], gbs=20, mbs=4)]),
    }
