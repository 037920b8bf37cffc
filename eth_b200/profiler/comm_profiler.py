"""Collective profiler: times all_gather / all_reduce / reduce_scatter / all_to_all over `tp` GPUs
for every distinct tensor size that appears in the op CSVs (reference:
eth/profiler/comm_profiler.py:85-147 timing, :194-207 size harvest, :157-171 output).

    python -m eth_b200.profiler.comm_profiler --prof-path out/ --prof-op-time-path out/ \
        --prof-tp-size 2 --prof-model-size 1_3B [--max-data-size 4096]

Writes `prim_gpt_<size>_<collective>_<n>gpus.csv` (`data_size(MB), time(ms)`) and a pickle. Sizes
above `--max-data-size` MB are not measured and recorded as 1e9 ms. Timing is CUDA events on the
launching stream, maximum over ranks.
"""
from __future__ import annotations

import argparse
import csv
import glob
import os
import pickle
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

PRIMS = ("all_gather", "all_reduce", "reduce_scatter", "all_to_all")
SKIPPED = 1.0e9


def harvest_sizes(op_time_path: str, model_size: str, tp: int):
    sizes = set()
    for path in glob.glob(os.path.join(op_time_path, f"gpt_{model_size}_mbs*_tp{tp}_algo*.csv")):
        with open(path, newline="") as f:
            rows = list(csv.reader(f))
        cols = [rows[0].index("input_size"), rows[0].index("output_size")]
        for r in rows[1:]:
            for c in cols:
                v = float(r[c])
                if v > 0:
                    sizes.add(round(v, 4))
    return sorted(sizes)


def time_collective(prim: str, numel: int, world: int, dtype, device, warmup: int, repeat: int) -> float:
    n = max(world, numel // world * world)
    x = torch.randn(n, device=device, dtype=dtype)
    if prim == "all_gather":
        out = torch.empty(n * world, device=device, dtype=dtype)
        fn = lambda: dist.all_gather_into_tensor(out, x)  # noqa: E731
    elif prim == "all_reduce":
        fn = lambda: dist.all_reduce(x)  # noqa: E731
    elif prim == "reduce_scatter":
        out = torch.empty(n // world, device=device, dtype=dtype)
        fn = lambda: dist.reduce_scatter_tensor(out, x)  # noqa: E731
    else:
        out = torch.empty_like(x)
        fn = lambda: dist.all_to_all_single(out, x)  # noqa: E731
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(repeat):
        fn()
    e.record()
    e.synchronize()
    t = torch.tensor([s.elapsed_time(e) / repeat], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _worker(rank, world, port, a):
    os.environ.update(MASTER_ADDR=os.environ.get("MASTER_ADDR", "127.0.0.1"), MASTER_PORT=str(port),
                      RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    dtype = torch.float32 if a.prof_dtype == "fp32" else torch.float16
    esize = 4 if a.prof_dtype == "fp32" else 2
    sizes = harvest_sizes(a.prof_op_time_path, a.prof_model_size, world)
    results = {}
    for prim in PRIMS:
        rows = []
        for mb_size in sizes:
            if mb_size > a.max_data_size:
                rows.append((mb_size, SKIPPED))
                continue
            numel = int(mb_size * 1024 * 1024 / esize)
            rows.append((mb_size, time_collective(prim, numel, world, dtype, device, a.prof_warmup_times, a.prof_repeat_times)))
        results[prim] = rows
        if rank == 0:
            with open(os.path.join(a.prof_path, f"prim_gpt_{a.prof_model_size}_{prim}_{world}gpus.csv"), "w", newline="") as f:
                w = csv.writer(f)
                w.writerow(["data_size(MB)", "time(ms)"])
                for s, t in rows:
                    w.writerow([s, f"{t:.5f}"])
    if rank == 0 and a.prof_cache_file:
        with open(a.prof_cache_file, "wb") as f:
            pickle.dump(results, f)
    dist.destroy_process_group()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--prof-path", required=True)
    ap.add_argument("--prof-cache-file", default=None)
    ap.add_argument("--prof-op-time-path", required=True)
    ap.add_argument("--prof-tp-size", type=int, required=True)
    ap.add_argument("--prof-model-name", default="gpt")
    ap.add_argument("--prof-model-size", required=True)
    ap.add_argument("--prof-warmup-times", type=int, default=5)
    ap.add_argument("--prof-repeat-times", type=int, default=20)
    ap.add_argument("--max-data-size", type=float, default=4096)
    ap.add_argument("--prof-dtype", default="fp16", choices=["fp16", "fp32"])
    a = ap.parse_args(argv)
    if a.prof_tp_size < 2:
        return
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(a.prof_tp_size, port, a), nprocs=a.prof_tp_size, join=True)


if __name__ == "__main__":
    main()
