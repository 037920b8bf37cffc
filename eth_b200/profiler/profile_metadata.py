"""`profile_metadata.json`, written atomically: schema_version 1, profile_status planned|complete,
model{name,size}, hardware, tp_sizes[], distributed{num_nodes,gpus_per_node,node_rank},
environment{python,torch,cuda} (reference: eth/profiler/profile_metadata.py:40-58)."""
from __future__ import annotations

import argparse
import json
import os
import platform
from pathlib import Path


def write_metadata(output: Path, status: str, model_size: str, hardware: str, tp_sizes, num_nodes=1,
                   gpus_per_node=1, node_rank=0, model_name="gpt"):
    if status not in ("planned", "complete"):
        raise ValueError("status must be planned or complete")
    try:
        import torch
        tv, cv = torch.__version__, torch.version.cuda
    except Exception:
        tv, cv = None, None
    meta = {"schema_version": 1, "profile_status": status, "model": {"name": model_name, "size": model_size},
            "hardware": hardware, "tp_sizes": sorted(int(t) for t in tp_sizes),
            "distributed": {"num_nodes": int(num_nodes), "gpus_per_node": int(gpus_per_node), "node_rank": int(node_rank)},
            "environment": {"python": platform.python_version(), "torch": tv, "cuda": cv}}
    output = Path(output)
    output.mkdir(parents=True, exist_ok=True)
    tmp = output / "profile_metadata.json.tmp"
    tmp.write_text(json.dumps(meta, indent=2) + "\n", encoding="utf-8")
    os.replace(tmp, output / "profile_metadata.json")
    return meta


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--output", type=Path, required=True)
    ap.add_argument("--status", required=True, choices=["planned", "complete"])
    ap.add_argument("--model", default="gpt")
    ap.add_argument("--model-size", required=True)
    ap.add_argument("--hardware", required=True)
    ap.add_argument("--tp-sizes", required=True, help="comma separated")
    ap.add_argument("--num-nodes", type=int, default=1)
    ap.add_argument("--gpus-per-node", type=int, default=1)
    ap.add_argument("--node-rank", type=int, default=0)
    a = ap.parse_args(argv)
    write_metadata(a.output, a.status, a.model_size, a.hardware, [int(t) for t in a.tp_sizes.split(",")],
                   a.num_nodes, a.gpus_per_node, a.node_rank, model_name=a.model)


if __name__ == "__main__":
    main()
