"""Convert a search result into the canonical `gpt_config.json`.

Accepts the hybrid `pipe[]` form written by this search, and the reference's legacy
single-pipeline JSON over the public 10-op-per-layer manifest or the legacy 13-op manifest
(the three score / softmax / dropout slots are dropped, eth/searching/config_adapter.py:43-63)."""
from __future__ import annotations

import argparse
import json
from pathlib import Path

from ..contract.config import normalize_flexpipe_config

TOPOLOGY_FIELDS = ("model_parallel_size_of_each_op", "data_parallel_size_of_each_op", "algo_of_each_op", "recompute_ops")
PIPE_ONLY = {"global_batch_size", "micro_batch_size", "num_stages", "num_gpus", "num_ops_in_each_stage",
             "checkpoint_activations", "resharding_stages", *TOPOLOGY_FIELDS}


def _legacy13_to_public_indices(num_layers):
    idx = [0]
    for layer in range(num_layers):
        b = 1 + layer * 13
        idx += [b, b + 1, b + 5, b + 6, b + 7, b + 8, b + 9, b + 10, b + 11, b + 12]
    tail = 1 + num_layers * 13
    return idx + [tail, tail + 1]


def convert(config):
    if isinstance(config.get("pipe"), list):
        return normalize_flexpipe_config(config)
    L = config.get("num_layers")
    if not isinstance(L, int) or L < 1:
        raise ValueError("search config num_layers must be positive")
    counts = config.get("num_ops_in_each_stage")
    if not isinstance(counts, list):
        raise ValueError("search config stage counts are invalid")
    total = sum(counts)
    if total == 3 + 10 * L:
        keep = list(range(total))
    elif total == 3 + 13 * L:
        keep = _legacy13_to_public_indices(L)
    else:
        raise ValueError("search config does not match a supported GPT manifest")
    stage_of = [s for s, n in enumerate(counts) for _ in range(n)]
    flat = {}
    for field in TOPOLOGY_FIELDS:
        vals = config.get(field)
        if not isinstance(vals, list) or len(vals) != len(counts):
            raise ValueError(f"{field} stage list is invalid")
        row = []
        for s, (v, n) in enumerate(zip(vals, counts)):
            if not isinstance(v, list) or len(v) != n:
                raise ValueError(f"{field} stage {s} length is invalid")
            row += v
        flat[field] = row
    kept_stage = [stage_of[i] for i in keep]
    stages = sorted(set(kept_stage))
    remap = {old: new for new, old in enumerate(stages)}
    pipe = {"global_batch_size": config["global_batch_size"], "micro_batch_size": config["micro_batch_size"],
            "num_stages": len(stages), "num_gpus": [config["num_gpus"][s] for s in stages],
            "num_ops_in_each_stage": [sum(1 for s in kept_stage if s == old) for old in stages],
            "checkpoint_activations": [config["checkpoint_activations"][s] for s in stages],
            "resharding_stages": [config["resharding_stages"][s] for s in stages]}
    for field in TOPOLOGY_FIELDS:
        grouped = [[] for _ in stages]
        for i, s in zip(keep, kept_stage):
            grouped[remap[s]].append(flat[field][i])
        pipe[field] = grouped
    out = {k: v for k, v in config.items() if k not in PIPE_ONLY}
    out["model_impl"] = "gpt"
    out["pipe"] = [pipe]
    return normalize_flexpipe_config(out)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", type=Path, required=True)
    ap.add_argument("--output", type=Path, required=True)
    a = ap.parse_args(argv)
    normalized = convert(json.loads(a.input.read_text(encoding="utf-8")))
    a.output.write_text(json.dumps(normalized, indent=2) + "\n", encoding="utf-8")


if __name__ == "__main__":
    main()
