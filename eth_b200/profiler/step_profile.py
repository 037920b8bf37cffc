"""Per-op time table of one training step (CUDA events around every op's forward and backward).

    python -m eth_b200.profiler.step_profile --size 1_3B --layers 24 --mbs 4 --microbatches 2 [--bf16]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29533 -m eth_b200.profiler.step_profile ...      (one stage, TP = number of ranks)

Prints one JSON line per (op, phase) with its share of the step, then host-side totals: wall time of
the step, device time between first and last event, and native launch count. The gap between the
sum of op times and the device time of the step is launch/host overhead.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch


def main(argv=None):
    from eth_b200.contract.config import GPT_SIZES, make_config, make_pipe, manifest_size
    from eth_b200.ops import native
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine

    ap = argparse.ArgumentParser()
    ap.add_argument("--size", default="1_3B")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--heads", type=int, default=None)
    ap.add_argument("--mbs", type=int, default=4)
    ap.add_argument("--microbatches", type=int, default=2)
    ap.add_argument("--bf16", action="store_true")
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--engine-args", default="", help="extra runtime flags, space separated (e.g. '--no-async-wgrad')")
    ap.add_argument("--all-ranks", action="store_true", help="print every rank's table, not only rank 0's")
    o = ap.parse_args(argv)
    m = dict(GPT_SIZES[o.size])
    if o.layers:
        m["num_layers"] = o.layers
    if o.heads:
        m["num_attention_heads"] = o.heads
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        import torch.distributed as dist
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = make_config([make_pipe([manifest_size(m["num_layers"])], [world], [1], gbs=o.mbs * o.microbatches, mbs=o.mbs)],
                      num_layers=m["num_layers"], hidden_size=m["hidden_size"],
                      num_attention_heads=m["num_attention_heads"], seq_length=m["seq_length"])
    argv2 = ["--bf16"] if o.bf16 else ["--fp16", "--loss-scale", "4096"]
    args = parse_args(argv2 + ["--hidden-dropout", "0.1"] + o.engine_args.split(), config=cfg, rank=rank, world_size=world)
    eng = TrainEngine(args)
    for _ in range(2):
        eng.train_step()
    torch.cuda.synchronize()
    # un-instrumented step
    l0 = native.launch_count()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    s.record()
    for _ in range(o.steps):
        eng.train_step(sync=False)
    e.record()
    host_ms = (time.perf_counter() - t0) * 1e3
    torch.cuda.synchronize()
    dev_ms = s.elapsed_time(e) / o.steps
    launches = (native.launch_count() - l0) // o.steps
    # instrumented step
    eng.stage.op_events = []
    eng.train_step(sync=False)
    table = eng.stage.op_time_table()
    eng.stage.op_events = None
    total = sum(table.values())
    if rank != 0 and not o.all_ranks:
        return
    for (name, phase), ms in sorted(table.items(), key=lambda kv: -kv[1]):
        print(json.dumps({"rank": rank, "op": name, "phase": phase, "ms": round(ms, 3), "share": round(ms / total, 4)}))
    print(json.dumps({"rank": rank, "summary": True, "step_device_ms": dev_ms, "host_enqueue_ms": host_ms / o.steps,
                      "sum_op_ms": total, "native_launches_per_step": launches,
                      "tokens_per_s": o.mbs * o.microbatches * m["seq_length"] / dev_ms * 1e3}))


if __name__ == "__main__":
    main()
