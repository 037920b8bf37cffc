#!/usr/bin/env python3
"""Compare the runtime evidence of a tensor-mode run and a block-mode run of the same config
(files `rank-<r>.json` written with --grad-sync-runtime-evidence-dir).

Required (reference: tools/validation/compare_runtime_evidence.py:116-213): same topology /
manifest / fragment hash; per rank and iteration the same total payload bytes and -- when both
runs saw the same gradients -- the same overall payload sha256; zero padding bytes; strictly
fewer collectives in block mode on every rank that synchronises more than one fragment; process
groups and scratch buffers stable over the run.
"""
import argparse
import json
from pathlib import Path


def load(dir_):
    out = {}
    for p in sorted(Path(dir_).glob("rank-*.json")):
        d = json.loads(p.read_text())
        out[d["global_rank"]] = d
    if not out:
        raise FileNotFoundError(f"no rank-*.json in {dir_}")
    return out


def compare_runs(tensor, block, check_payload_hash=True):
    problems = []
    if set(tensor) != set(block):
        return [f"rank sets differ: {sorted(tensor)} vs {sorted(block)}"]
    for r in sorted(tensor):
        t, b = tensor[r], block[r]
        if t["sync_mode"] != "tensor" or b["sync_mode"] != "block":
            problems.append(f"rank {r}: expected tensor vs block runs, got {t['sync_mode']} vs {b['sync_mode']}")
        for key in ("global_topology_hash", "global_manifest_hash", "global_fragment_hash"):
            if t[key] != b[key]:
                problems.append(f"rank {r}: {key} differs")
        for name, run in (("tensor", t), ("block", b)):
            if run["padding_payload_bytes"] != 0:
                problems.append(f"rank {r}: {name} run has padding bytes")
            for flag in ("process_group_count_stable", "process_group_creation_count_stable", "scratch_stable"):
                if not run[flag]:
                    problems.append(f"rank {r}: {name} run {flag} is false")
        if len(t["iterations"]) != len(b["iterations"]):
            problems.append(f"rank {r}: iteration counts differ")
            continue
        for it_t, it_b in zip(t["iterations"], b["iterations"]):
            i = it_t["iteration"]
            if it_t["payload_bytes"] != it_b["payload_bytes"]:
                problems.append(f"rank {r} iter {i}: payload bytes {it_t['payload_bytes']} vs {it_b['payload_bytes']}")
            if it_t["collective_count"] > 1 and not it_b["collective_count"] < it_t["collective_count"]:
                problems.append(f"rank {r} iter {i}: block mode issued {it_b['collective_count']} collectives, "
                                f"tensor mode {it_t['collective_count']}")
            if check_payload_hash and it_t["packed_payload_sha256"] != it_b["packed_payload_sha256"]:
                problems.append(f"rank {r} iter {i}: packed payload hashes differ")
    return problems


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tensor", required=True)
    ap.add_argument("--block", required=True)
    ap.add_argument("--skip-payload-hash", action="store_true",
                    help="bucket order differs between modes only if fragment order does; skip the byte-level check")
    a = ap.parse_args(argv)
    problems = compare_runs(load(a.tensor), load(a.block), not a.skip_payload_hash)
    print(json.dumps({"consistent": not problems, "problems": problems[:20]}, indent=1))
    return 1 if problems else 0


if __name__ == "__main__":
    raise SystemExit(main())
