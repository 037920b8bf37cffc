"""Gate between profiling and search: check a profile directory and a node description, write
`node_info.json`, `device_info.json` and `search_contract.json`, and print the four lines the
launcher reads (hardware label, max TP, total GPUs, node_info JSON).

The checks are data: a schema for the node description (`NODE_ENTRY`, `DEVICE_ENTRY`), a list of
metadata rules (`METADATA_RULES`) and a generator of the record files a searchable profile must
contain (`expected_records`), each walked by a small interpreter. What is checked follows the
reference (eth/searching/profile_validation.py:36-44 TP coverage, :47-79 node description,
:114-136 records, :169-191 outputs).
"""
from __future__ import annotations

import argparse
import csv
import json
from pathlib import Path
from typing import Callable, Iterator, NamedTuple

from .profile_db import COLLECTIVES, OP_HEADER

MICRO_BATCH_SIZES = (1, 2, 4, 8)
ALGORITHMS = (0, 1)
COLLECTIVE_HEADER = ["data_size(MB)", "time(ms)"]


class ProfileError(SystemExit):
    def __init__(self, message: str):
        super().__init__(f"profile validation failed: {message}")


# ------------------------------------------------------------------------------------------
# node description schema
# ------------------------------------------------------------------------------------------
def _text(v):
    return isinstance(v, str) and bool(v)


def _count(v):
    return isinstance(v, int) and not isinstance(v, bool) and v >= 1


def _amount(v):
    return isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0


# field -> (predicate, what the message says when the predicate fails)
NODE_ENTRY = {"GPU": (_text, "must be a non-empty string"), "GPU_NUM": (_count, "must be positive"),
              "NODE_NUM": (_count, "must be positive")}
DEVICE_ENTRY = {"memory": (_amount, "must be positive"), "intra_bandwidth": (_amount, "must be positive"),
                "TFLOPS": (_amount, "must be positive")}


def _check_table(table, name: str, schema, missing_is_invalid: bool) -> None:
    for key, entry in table.items():
        if not isinstance(entry, dict):
            raise ProfileError(f"{name}[{key}] must be an object")
        for fieldname, (accept, complaint) in schema.items():
            if fieldname not in entry and not missing_is_invalid:
                raise ProfileError(f"{name}[{key}] is missing {fieldname}")
            if not accept(entry.get(fieldname)):
                raise ProfileError(f"{name}[{key}].{fieldname} {complaint}")


def validate_node_description(description):
    if not isinstance(description, dict):
        raise ProfileError("node description must be a JSON object")
    tables = {}
    for name in ("node_info", "device_info"):
        table = description.get(name)
        if not isinstance(table, dict) or not table:
            raise ProfileError(f"node description requires non-empty {name}")
        tables[name] = table
    _check_table(tables["node_info"], "node_info", NODE_ENTRY, missing_is_invalid=False)
    for entry in tables["node_info"].values():
        if entry["GPU"] not in tables["device_info"]:
            raise ProfileError(f"device_info is missing hardware {entry['GPU']}")
    _check_table(tables["device_info"], "device_info", DEVICE_ENTRY, missing_is_invalid=True)
    return tables["node_info"], tables["device_info"]


def required_tp_sizes(model_size: str, node_info) -> list:
    """Powers of two up to min(GPUs of the largest node, 8), and up to 4 for the 350M model."""
    limit = min(max(e["GPU_NUM"] for e in node_info.values()), 4 if model_size == "350M" else 8)
    return [1 << k for k in range(limit.bit_length()) if (1 << k) <= limit]


# ------------------------------------------------------------------------------------------
# metadata rules: (test on (metadata, context), message)
# ------------------------------------------------------------------------------------------
class Context(NamedTuple):
    model_size: str
    hardware_labels: frozenset
    tp_sizes: tuple


METADATA_RULES = (
    (lambda m, c: m.get("schema_version") == 1, lambda c: "profile schema_version must be 1"),
    (lambda m, c: m.get("profile_status") == "complete",
     lambda c: "profile_status must be complete; planned dry-run data cannot be searched"),
    (lambda m, c: (m.get("model") or {}).get("name") == "gpt" and (m.get("model") or {}).get("size") == c.model_size,
     lambda c: f"profile model size does not match requested {c.model_size}"),
    (lambda m, c: c.hardware_labels == {m.get("hardware")},
     lambda c: "profile hardware does not match node description; one canonical profile currently supports "
               "one hardware label"),
    (lambda m, c: isinstance(m.get("tp_sizes"), list) and set(c.tp_sizes) <= set(m["tp_sizes"]),
     lambda c: f"profile TP coverage must include {list(c.tp_sizes)}"),
)


# ------------------------------------------------------------------------------------------
# record files
# ------------------------------------------------------------------------------------------
def _table_with_header(header) -> Callable[[Path], None]:
    def check(path: Path) -> None:
        with path.open(newline="", encoding="utf-8") as f:
            rows = csv.reader(f)
            first, second = next(rows), next(rows)
        if first != header or not second:
            raise ProfileError(f"invalid profile record schema: {path.name}")
    return check


def _numeric_matrix(path: Path) -> None:
    with path.open(newline="", encoding="utf-8") as f:
        rows = list(csv.reader(f))
    if len(rows) < 2 or len(rows[0]) < 2:
        raise ValueError("expected size and bandwidth rows")
    if len({len(r) for r in rows}) != 1:
        raise ValueError("rows have inconsistent widths")
    for r in rows:
        for cell in r:
            float(cell)


def expected_records(model_size: str, tp_sizes, inter_node: bool) -> Iterator[tuple]:
    """(file name, checker, message prefix on a malformed file) for every record a search needs."""
    for mbs in MICRO_BATCH_SIZES:
        for tp in tp_sizes:
            for algo in ALGORITHMS:
                yield f"gpt_{model_size}_mbs{mbs}_tp{tp}_algo{algo}.csv", _table_with_header(OP_HEADER), "invalid profile record"
    for tp in tp_sizes:
        if tp > 1:
            for prim in COLLECTIVES:
                yield (f"prim_gpt_{model_size}_{prim}_{tp}gpus.csv", _table_with_header(COLLECTIVE_HEADER),
                       "invalid profile record")
    yield "p2p_intra_node.csv", _numeric_matrix, "invalid P2P profile record"
    if inter_node:
        yield "p2p_inter_node.csv", _numeric_matrix, "invalid P2P profile record"


def validate_records(profile_dir: Path, model_size, tp_sizes, need_inter_node) -> None:
    for name, check, prefix in expected_records(model_size, tp_sizes, need_inter_node):
        path = profile_dir / name
        if not path.is_file():
            raise ProfileError(f"required profile record is missing: {name}")
        try:
            check(path)
        except (OSError, StopIteration, ValueError, csv.Error) as err:
            raise ProfileError(f"{prefix} {name}: {err}") from None


# ------------------------------------------------------------------------------------------
def load_json(path: Path, label: str):
    if not path.is_file():
        raise ProfileError(f"missing {label}: {path}")
    try:
        return json.loads(path.read_text(encoding="utf-8"))
    except (OSError, json.JSONDecodeError) as err:
        raise ProfileError(f"invalid {label}: {err}") from None


def _write_json(path: Path, value) -> None:
    path.write_text(json.dumps(value, indent=2) + "\n", encoding="utf-8")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile-dir", type=Path, required=True)
    ap.add_argument("--model-size", required=True)
    ap.add_argument("--node-description", type=Path, required=True)
    ap.add_argument("--output", type=Path, required=True)
    a = ap.parse_args(argv)
    metadata = load_json(a.profile_dir / "profile_metadata.json", "profile metadata")
    node_info, device_info = validate_node_description(load_json(a.node_description, "node description"))
    tp_sizes = required_tp_sizes(a.model_size, node_info)
    ctx = Context(a.model_size, frozenset(e["GPU"] for e in node_info.values()), tuple(tp_sizes))
    for holds, message in METADATA_RULES:
        if not holds(metadata, ctx):
            raise ProfileError(message(ctx))
    node_count = sum(e["NODE_NUM"] for e in node_info.values())
    validate_records(a.profile_dir, a.model_size, tp_sizes, node_count > 1)
    contract = {"hardware": metadata["hardware"], "max_tp": max(tp_sizes), "node_count": node_count,
                "total_gpus": sum(e["GPU_NUM"] * e["NODE_NUM"] for e in node_info.values()), "node_info": node_info}
    a.output.mkdir(parents=True, exist_ok=True)
    for name, value in (("node_info.json", node_info), ("device_info.json", device_info),
                        ("search_contract.json", contract)):
        _write_json(a.output / name, value)
    for line in (contract["hardware"], contract["max_tp"], contract["total_gpus"],
                 json.dumps(node_info, separators=(",", ":"))):
        print(line)


if __name__ == "__main__":
    main()
