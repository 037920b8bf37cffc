"""The `gpt_config.json` contract: canonical form of a heterogeneous-pipeline (HPP) GPT config.

Same public schema as the reference normalizer (eth/runtime/megatron/config_normalization.py):
allowed top-level keys (:38-55) and per-pipeline keys (:57-77); the 3 + 10*L op manifest with a
sha256 hash (:91-136); every topology field accepted per stage (`*_of_each_stage`) or per op
(`*_of_each_op`), constant inside a stage (:209-246); TP in {1,2,4,6,8}, CP == 1,
num_gpus == TP*DP*CP, batch divisibility, hidden/heads divisible by TP (:272-311, 372-386); and the
derived `world_size`, `total_gbs`, `pipeline_sample_offsets`, `topology_fingerprint`, `config_hash`
(:387-432). Hashes are sha256 over compact sorted-key JSON, so a config normalized here and by the
reference carries the same `config_hash`.

A pipeline is read by `_PipelineReader`, which runs the clauses of the contract in a fixed order;
the two spellings of a topology field are handled by `TopologyField`. The output is plain
JSON-serialisable dicts because that *is* the contract.
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
# The older 13-op layer: attention is four ops (scores, softmax, dropout, context) instead of one
# fused flash-attention op (reference: eth/searching/model_ops.py:10-43,
# eth/runtime/megatron/model/flex_ops.py:1144-1519).
LEGACY_LAYER_OPS = (
    "enc-1st-layernorm", "enc-attention-qkv", "enc-attention-score", "enc-attention-softmax",
    "enc-attention-dropout", "enc-attention-context", "enc-attention-dense", "enc-post-attention-dropout",
    "enc-2nd-layernorm", "enc-MLP-GEMM-1", "enc-MLP-gelu", "enc-MLP-GEMM-2", "enc-post-MLP-dropout",
)
FIRST_OP = "encoder-embedding"
TAIL_OPS = ("final-layernorm", "gpt-post-process")
MODEL_IMPLS = {
    "gpt": {"id": "gpt", "ops_per_layer": len(LAYER_OPS), "layer_schema": LAYER_OPS},
    "gpt-legacy13": {"id": "gpt-legacy13", "ops_per_layer": len(LEGACY_LAYER_OPS), "layer_schema": LEGACY_LAYER_OPS},
}

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


# ------------------------------------------------------------------------------------------
# one pipeline: a reader object that turns the raw dict into the canonical one, clause by clause
# ------------------------------------------------------------------------------------------
class TopologyField:
    """A per-op topology field that may be written per stage (`<stem>_of_each_stage`, one value per
    stage) or per op (`<stem>_of_each_op`, one list per stage). Canonical form: per op. Both
    spellings, if present, must say the same; values must not change inside a stage."""

    def __init__(self, stem: str, default=None):
        self.stem, self.default = stem, default
        self.brief_key, self.full_key = f"{stem}_of_each_stage", f"{stem}_of_each_op"

    def _expanded_brief(self, pipe, stage_ops):
        brief = pipe.get(self.brief_key)
        if brief is None:
            if self.full_key in pipe or self.default is None:
                return None
            brief = [self.default] * len(stage_ops)
        if not isinstance(brief, list) or len(brief) != len(stage_ops):
            raise ConfigError(f"{self.brief_key} stage list length must equal num_stages")
        return [[value] * count for value, count in zip(brief, stage_ops)]

    def _checked_full(self, pipe, stage_ops):
        full = pipe.get(self.full_key)
        if full is None:
            return None
        if not isinstance(full, list) or len(full) != len(stage_ops):
            raise ConfigError(f"{self.full_key} stage list length must equal num_stages")
        for stage, (values, count) in enumerate(zip(full, stage_ops)):
            if not isinstance(values, list) or len(values) != count:
                raise ConfigError(f"{self.full_key} stage {stage} length must equal its op count")
            if any(v != values[0] for v in values):
                raise ConfigError(f"intra-stage constancy violated for {self.full_key} at stage {stage}")
        return [list(values) for values in full]

    def read(self, pipe, stage_ops):
        brief, full = self._expanded_brief(pipe, stage_ops), self._checked_full(pipe, stage_ops)
        if brief is None and full is None:
            raise ConfigError(f"missing {self.brief_key} or {self.full_key}")
        if brief is not None and full is not None and brief != full:
            raise ConfigError(f"brief and expanded {self.stem} values conflict")
        return full if full is not None else brief


TOPOLOGY_FIELDS = (TopologyField("model_parallel_size"), TopologyField("data_parallel_size"),
                   TopologyField("context_parallel_size", default=1), TopologyField("algo"))


class _PipelineReader:
    """Reads one raw pipeline dict. `canonical()` runs the clauses of the contract in a fixed order
    (the first violated clause is the one reported) and returns the canonical dict."""

    def __init__(self, raw: Dict[str, Any], index: int, manifest_ops: int):
        self.raw, self.index, self.manifest_ops = copy.deepcopy(raw), index, manifest_ops
        self.stages = 0
        self.stage_ops: List[int] = []
        self.per_op: Dict[str, list] = {}

    # -- helpers
    def _per_stage(self, key):
        value = self.raw.get(key)
        if not isinstance(value, list) or len(value) != self.stages:
            raise ConfigError(f"{key} stage list length must equal num_stages")
        return value

    def _degree(self, stem):
        return [values[0] for values in self.per_op[f"{stem}_of_each_op"]]

    # -- clauses
    def read_stage_layout(self):
        self.stages = self.raw.get("num_stages")
        if not _is_pos_int(self.stages):
            raise ConfigError(f"pipeline {self.index} num_stages must be positive")
        self.stage_ops = self._per_stage("num_ops_in_each_stage")
        if not all(_is_pos_int(n) for n in self.stage_ops):
            raise ConfigError("num_ops_in_each_stage values must be positive integers")
        if sum(self.stage_ops) != self.manifest_ops:
            raise ConfigError(f"manifest size mismatch in pipeline {self.index}: expected {self.manifest_ops}, "
                              f"got {sum(self.stage_ops)}")

    def read_topology_fields(self):
        for f in TOPOLOGY_FIELDS:
            self.per_op[f.full_key] = f.read(self.raw, self.stage_ops)

    def check_degrees(self):
        tp, dp, cp = self._degree("model_parallel_size"), self._degree("data_parallel_size"), self._degree("context_parallel_size")
        for stage, c in enumerate(cp):
            if c != 1:
                raise ConfigError(f"context parallel stage {stage} must be 1 for block-wise sync")
        for label, values in (("TP", tp), ("DP", dp), ("CP", cp)):
            if not all(_is_pos_int(v) for v in values):
                raise ConfigError(f"{label} values must be positive integers")
        for stage, t in enumerate(tp):
            if t not in SUPPORTED_TP:
                raise ConfigError(f"unsupported TP value {t} in pipeline {self.index} stage {stage}; supported TP "
                                  "values are " + ", ".join(map(str, SUPPORTED_TP)))
        for stage, (gpus, t, d, c) in enumerate(zip(self._per_stage("num_gpus"), tp, dp, cp)):
            if gpus != t * d * c:
                raise ConfigError(f"stage product mismatch in pipeline {self.index} stage {stage}: "
                                  f"num_gpus={gpus}, TP*DP*CP={t * d * c}")

    def check_batches(self):
        mbs, gbs = self.raw.get("micro_batch_size"), self.raw.get("global_batch_size")
        for name, value in (("micro_batch_size", mbs), ("global_batch_size", gbs)):
            if not _is_pos_int(value):
                raise ConfigError(f"{name} must be a positive integer")
        if gbs % mbs:
            raise ConfigError("micro batch divisibility requires GBS % micro_batch_size == 0")
        for stage, d in enumerate(self._degree("data_parallel_size")):
            if mbs % d:
                raise ConfigError(f"micro batch divisibility failed for pipeline {self.index} stage {stage}: "
                                  "micro_batch_size % DP != 0")

    def check_recompute(self):
        for stage, (flags, count) in enumerate(zip(self._per_stage("recompute_ops"), self.stage_ops)):
            if not isinstance(flags, list) or len(flags) != count:
                raise ConfigError(f"recompute_ops stage {stage} length must equal its op count")

    CLAUSES = (read_stage_layout, read_topology_fields, check_degrees, check_batches, check_recompute)

    def canonical(self) -> Dict[str, Any]:
        for clause in self.CLAUSES:
            clause(self)
        out = {"pipeline_index": self.index, "global_batch_size": self.raw["global_batch_size"],
               "micro_batch_size": self.raw["micro_batch_size"], "num_stages": self.stages,
               "num_gpus": list(self.raw["num_gpus"]), "num_ops_in_each_stage": list(self.stage_ops)}
        for key in ("checkpoint_activations", "resharding_stages"):
            out[key] = list(self._per_stage(key))
        out["recompute_ops"] = self.raw["recompute_ops"]
        out.update(self.per_op)
        return out


def _normalize_pipeline(src: Dict[str, Any], index: int, n_ops: int) -> Dict[str, Any]:
    return _PipelineReader(src, index, n_ops).canonical()


def _reject_unknown(mapping, allowed, what):
    extra = sorted(set(mapping) - allowed)
    if extra:
        raise ConfigError(f"{what}: {', '.join(extra)}")


FINGERPRINT_KEYS = ("num_gpus", "num_ops_in_each_stage", "model_parallel_size_of_each_op",
                    "data_parallel_size_of_each_op", "context_parallel_size_of_each_op")


def normalize_flexpipe_config(config: Dict[str, Any], world_size: Optional[int] = None) -> Dict[str, Any]:
    """Unique canonical representation of an HPP GPT config (raises ConfigError on violations)."""
    if not isinstance(config, dict):
        raise ConfigError("config must be a mapping")
    _reject_unknown(config, TOP_LEVEL_KEYS, "unknown top-level config field(s)")
    raw_pipes = config.get("pipe")
    if not isinstance(raw_pipes, list) or not raw_pipes:
        raise ConfigError("config must contain at least one pipeline")
    op_totals = []
    for i, raw in enumerate(raw_pipes):
        if not isinstance(raw, dict):
            raise ConfigError(f"pipeline {i} must be a mapping")
        _reject_unknown(raw, PIPE_KEYS, f"pipeline {i} has unknown field(s)")
        counts = raw.get("num_ops_in_each_stage")
        if not isinstance(counts, list) or not counts:
            raise ConfigError(f"pipeline {i} is missing num_ops_in_each_stage")
        op_totals.append(sum(counts))
    impl = _resolve_model_impl(config, op_totals)
    manifest = build_manifest(impl, config["num_layers"])
    pipes = [_normalize_pipeline(raw, i, len(manifest["ordered_ops"])) for i, raw in enumerate(raw_pipes)]

    hidden, heads = config.get("hidden_size"), config.get("num_attention_heads")
    for pi, pipe in enumerate(pipes):
        for si, per_op in enumerate(pipe["model_parallel_size_of_each_op"]):
            divisible = isinstance(hidden, int) and isinstance(heads, int) and hidden % per_op[0] == 0 and heads % per_op[0] == 0
            if not divisible:
                raise ConfigError(f"TP constraint failed in pipeline {pi} stage {si}: hidden_size={hidden}, "
                                  f"num_attention_heads={heads}, TP={per_op[0]}")
    world = sum(sum(p["num_gpus"]) for p in pipes)
    if world_size is not None and world_size != world:
        raise ConfigError(f"world size mismatch: expected {world}, got {world_size}")
    batch_sizes = [p["global_batch_size"] for p in pipes]
    offsets = [sum(batch_sizes[:i]) for i in range(len(batch_sizes))]

    out = {k: copy.deepcopy(v) for k, v in config.items() if k not in ("pipe", "model_impl")}
    out.update(model_impl=impl, manifest=manifest, pipe=pipes, world_size=world, total_gbs=sum(batch_sizes),
               pipeline_sample_offsets=offsets)
    out["topology_fingerprint"] = canonical_hash(
        {"world_size": world, "pipelines": [{k: p[k] for k in FINGERPRINT_KEYS} for p in pipes]})
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
