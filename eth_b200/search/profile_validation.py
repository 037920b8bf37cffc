"""Validate a profile directory and a node description before a search, write `node_info.json`,
`device_info.json` and `search_contract.json`, and print the four-line contract the launcher reads
(hardware label, max TP, total GPUs, node_info JSON) -- reference:
eth/searching/profile_validation.py:36-44 TP coverage, :47-79 node description, :114-136 records,
:169-191 outputs."""
from __future__ import annotations

import argparse
import csv
import json
from pathlib import Path

from .profile_db import COLLECTIVES, OP_HEADER

MICRO_BATCH_SIZES = (1, 2, 4, 8)
ALGORITHMS = (0, 1)


def fail(msg):
    raise SystemExit(f"profile validation failed: {msg}")


def load_json(path: Path, label: str):
    if not path.is_file():
        fail(f"missing {label}: {path}")
    try:
        return json.loads(path.read_text(encoding="utf-8"))
    except (OSError, json.JSONDecodeError) as e:
        fail(f"invalid {label}: {e}")


def required_tp_sizes(model_size, node_info):
    most = max(e["GPU_NUM"] for e in node_info.values())
    cap = min(most, 4 if model_size == "350M" else 8)
    out, v = [], 1
    while v <= cap:
        out.append(v)
        v *= 2
    return out


def validate_node_description(desc):
    if not isinstance(desc, dict):
        fail("node description must be a JSON object")
    node_info, device_info = desc.get("node_info"), desc.get("device_info")
    if not isinstance(node_info, dict) or not node_info:
        fail("node description requires non-empty node_info")
    if not isinstance(device_info, dict) or not device_info:
        fail("node description requires non-empty device_info")
    for key, e in node_info.items():
        if not isinstance(e, dict):
            fail(f"node_info[{key}] must be an object")
        for f in ("GPU", "GPU_NUM", "NODE_NUM"):
            if f not in e:
                fail(f"node_info[{key}] is missing {f}")
        if not isinstance(e["GPU"], str) or not e["GPU"]:
            fail(f"node_info[{key}].GPU must be a non-empty string")
        for f in ("GPU_NUM", "NODE_NUM"):
            if not isinstance(e[f], int) or e[f] < 1:
                fail(f"node_info[{key}].{f} must be positive")
        if e["GPU"] not in device_info:
            fail(f"device_info is missing hardware {e['GPU']}")
    for hw, e in device_info.items():
        if not isinstance(e, dict):
            fail(f"device_info[{hw}] must be an object")
        for f in ("memory", "intra_bandwidth", "TFLOPS"):
            v = e.get(f)
            if not isinstance(v, (int, float)) or v <= 0:
                fail(f"device_info[{hw}].{f} must be positive")
    return node_info, device_info


def _check_csv(path: Path, header):
    if not path.is_file():
        fail(f"required profile record is missing: {path.name}")
    try:
        with path.open(newline="", encoding="utf-8") as f:
            r = csv.reader(f)
            got = next(r)
            row = next(r)
    except (OSError, StopIteration, csv.Error) as e:
        fail(f"invalid profile record {path.name}: {e}")
    if got != header or not row:
        fail(f"invalid profile record schema: {path.name}")


def _check_p2p(path: Path):
    if not path.is_file():
        fail(f"required profile record is missing: {path.name}")
    try:
        with path.open(newline="", encoding="utf-8") as f:
            rows = list(csv.reader(f))
        if len(rows) < 2 or len(rows[0]) < 2:
            raise ValueError("expected size and bandwidth rows")
        if any(len(r) != len(rows[0]) for r in rows[1:]):
            raise ValueError("rows have inconsistent widths")
        for r in rows:
            for v in r:
                float(v)
    except (OSError, ValueError, csv.Error) as e:
        fail(f"invalid P2P profile record {path.name}: {e}")


def validate_records(profile_dir: Path, model_size, tp_sizes, need_inter_node):
    for mbs in MICRO_BATCH_SIZES:
        for tp in tp_sizes:
            for algo in ALGORITHMS:
                _check_csv(profile_dir / f"gpt_{model_size}_mbs{mbs}_tp{tp}_algo{algo}.csv", OP_HEADER)
    for tp in tp_sizes:
        if tp == 1:
            continue
        for prim in COLLECTIVES:
            _check_csv(profile_dir / f"prim_gpt_{model_size}_{prim}_{tp}gpus.csv", ["data_size(MB)", "time(ms)"])
    _check_p2p(profile_dir / "p2p_intra_node.csv")
    if need_inter_node:
        _check_p2p(profile_dir / "p2p_inter_node.csv")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile-dir", type=Path, required=True)
    ap.add_argument("--model-size", required=True)
    ap.add_argument("--node-description", type=Path, required=True)
    ap.add_argument("--output", type=Path, required=True)
    a = ap.parse_args(argv)
    meta = load_json(a.profile_dir / "profile_metadata.json", "profile metadata")
    node_info, device_info = validate_node_description(load_json(a.node_description, "node description"))
    if meta.get("schema_version") != 1:
        fail("profile schema_version must be 1")
    if meta.get("profile_status") != "complete":
        fail("profile_status must be complete; planned dry-run data cannot be searched")
    model = meta.get("model", {})
    if model.get("name") != "gpt" or model.get("size") != a.model_size:
        fail(f"profile model size does not match requested {a.model_size}")
    labels = {e["GPU"] for e in node_info.values()}
    hw = meta.get("hardware")
    if labels != {hw}:
        fail("profile hardware does not match node description; one canonical profile currently supports one hardware label")
    tp_sizes = required_tp_sizes(a.model_size, node_info)
    covered = meta.get("tp_sizes")
    if not isinstance(covered, list) or any(t not in covered for t in tp_sizes):
        fail(f"profile TP coverage must include {tp_sizes}")
    nodes = sum(e["NODE_NUM"] for e in node_info.values())
    validate_records(a.profile_dir, a.model_size, tp_sizes, nodes > 1)
    a.output.mkdir(parents=True, exist_ok=True)
    (a.output / "node_info.json").write_text(json.dumps(node_info, indent=2) + "\n", encoding="utf-8")
    (a.output / "device_info.json").write_text(json.dumps(device_info, indent=2) + "\n", encoding="utf-8")
    contract = {"hardware": hw, "max_tp": max(tp_sizes), "node_count": nodes,
                "total_gpus": sum(e["GPU_NUM"] * e["NODE_NUM"] for e in node_info.values()), "node_info": node_info}
    (a.output / "search_contract.json").write_text(json.dumps(contract, indent=2) + "\n", encoding="utf-8")
    print(hw)
    print(max(tp_sizes))
    print(contract["total_gpus"])
    print(json.dumps(node_info, separators=(",", ":")))


if __name__ == "__main__":
    main()
