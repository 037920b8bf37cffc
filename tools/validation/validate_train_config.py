#!/usr/bin/env python3
"""CPU-only pre-flight of a GPT HPP config: normalise it against the world size, lay out the
canonical topology and print its fingerprint. Runs before any CUDA or distributed set-up."""
import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from eth_b200.contract.config import normalize_flexpipe_config  # noqa: E402
from eth_b200.parallel.grad_sync.topology import build_canonical_topology  # noqa: E402

# (what must hold for a trainable public config, message when it does not)
REQUIREMENTS = (
    (lambda cfg, topo, world: cfg["model_name"] == "gpt", "only GPT configs are supported"),
    (lambda cfg, topo, world: cfg["model_impl"] == "gpt", "public training requires model_impl gpt"),
    (lambda cfg, topo, world: topo.world_size == world, "canonical topology world size mismatch"),
)


def inspect(config_path: Path, world_size: int):
    """(normalised config, topology); raises ValueError / OSError / KeyError with the reason."""
    raw = json.loads(config_path.read_text(encoding="utf-8"))
    cfg = normalize_flexpipe_config(raw, world_size=world_size)
    topo = build_canonical_topology(cfg)
    for holds, message in REQUIREMENTS:
        if not holds(cfg, topo, world_size):
            raise ValueError(message)
    return cfg, topo


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", type=Path, required=True)
    ap.add_argument("--world-size", type=int, required=True)
    ap.add_argument("--grad-sync-mode", choices=("tensor", "block"), required=True)
    opts = ap.parse_args(argv)
    try:
        cfg, topo = inspect(opts.config, opts.world_size)
    except (OSError, ValueError, KeyError) as err:    # JSONDecodeError is a ValueError
        print(f"config validation failed: {err}", file=sys.stderr)
        return 1
    summary = {"model_impl": cfg["model_impl"], "world_size": topo.world_size,
               "grad_sync_mode": opts.grad_sync_mode, "topology": topo.fingerprint}
    print("config validated: " + " ".join(f"{k}={v}" for k, v in summary.items()))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
