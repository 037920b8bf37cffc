#!/usr/bin/env python3
"""Validate a GPT HPP config before CUDA or distributed set-up: normalize it against the world
size, build the canonical topology and print its fingerprint (CPU only)."""
import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from eth_b200.contract.config import normalize_flexpipe_config  # noqa: E402
from eth_b200.parallel.grad_sync.topology import build_canonical_topology  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=Path, required=True)
    ap.add_argument("--world-size", type=int, required=True)
    ap.add_argument("--grad-sync-mode", choices=("tensor", "block"), required=True)
    a = ap.parse_args(argv)
    try:
        normalized = normalize_flexpipe_config(json.loads(a.config.read_text(encoding="utf-8")), world_size=a.world_size)
        if normalized["model_name"] != "gpt":
            raise ValueError("only GPT configs are supported")
        if normalized["model_impl"] != "gpt":
            raise ValueError("public training requires model_impl gpt")
        topo = build_canonical_topology(normalized)
        if topo.world_size != a.world_size:
            raise ValueError("canonical topology world size mismatch")
    except (OSError, ValueError, KeyError, json.JSONDecodeError) as e:
        print(f"config validation failed: {e}", file=sys.stderr)
        return 1
    print(f"config validated: model_impl={normalized['model_impl']} world_size={topo.world_size} "
          f"grad_sync_mode={a.grad_sync_mode} topology={topo.fingerprint}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
