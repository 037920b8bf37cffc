"""Micro-benchmark of the fused tensor-parallel kernels against their library baselines.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29533 -m eth_b200.profiler.fused_collective_bench [--tokens 8192] [--hidden 2048]
        [--sweep-k 64,1024,2048,4096,8192]

For the GEMM shapes of one transformer layer at this tensor-parallel width it times
  * GEMM + all-reduce      (row-parallel forward, column-parallel data gradient),
  * GEMM + reduce-scatter  (the same linears in sequence-parallel form),
  * all-gather + GEMM      (column-parallel forward in sequence-parallel form),
each as ONE fused kernel and as "GEMM kernel + NCCL collective", with CUDA events on the launching
stream after warm-up, maximum over ranks, and prints one JSON line per case with the roofline
fraction: target time = max(FLOPs / measured GEMM peak, bytes over NVLink / 770 GB/s per direction).
`--sweep-k` instead times the fused GEMM + all-reduce at [tokens, hidden] for a list of reduction
lengths: with almost no math (K = 64) the time is the communication floor of the kernel, and the K
at which the time starts to grow is where it turns compute-bound.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0   # measured peer-copy bandwidth per direction per GPU


def main(argv=None):
    from eth_b200 import ops
    from eth_b200.ops import native
    from eth_b200.parallel.fused_tp import FusedTPBackend
    from eth_b200.profiler.kernel_bench import _peaks

    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--repeat", type=int, default=20)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--sweep-k", default=None, help="comma-separated reduction lengths (per rank) for the K sweep")
    a = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float16
    _, peak_tflops, src = _peaks()
    M, H = a.tokens, a.hidden
    be = FusedTPBackend(tuple(range(world)), rank, None, dev, max_tokens=M, hidden=4 * H, dtype=dt)

    def timeit(fn):
        for _ in range(5):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(a.repeat):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / a.repeat], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() * 1e3   # microseconds

    def report(kind, tag, n, k, fused_us, base_us, gemm_us, link_bytes):
        flops = 2.0 * M * n * k
        target = max(flops / (peak_tflops * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e6
        if rank == 0:
            print(json.dumps({"kernel": kind, "case": tag, "world": world, "M": M, "N": n, "K": k,
                              "fused_us": round(fused_us, 1), "gemm_plus_nccl_us": round(base_us, 1),
                              "gemm_only_us": round(gemm_us, 1), "roofline_target_us": round(target, 1),
                              "frac_of_roofline": round(target / fused_us, 3), "peak": src}), flush=True)

    esz = 2
    frac = (world - 1) / world
    if a.sweep_k:
        for k in [int(v) for v in a.sweep_k.split(",")]:
            x = torch.randn(M, k, device=dev, dtype=dt)
            w = torch.randn(H, k, device=dev, dtype=dt) * 0.05
            out = torch.empty(M, H, device=dev, dtype=dt)
            report("gemm_allreduce", f"K sweep, {2 * frac * M * H * esz / 2 ** 20:.0f} MiB each way", H, k,
                   timeit(lambda: be.gemm_all_reduce(x, w)), float("nan"), timeit(lambda: ops.gemm(x, w, out=out)),
                   2 * frac * M * H * esz)
        native.check_status()
        be.close()
        dist.destroy_process_group()
        return
    for (n, k, b_mn, tag) in [(H, H // world, False, "attention-dense fwd"), (H, 4 * H // world, False, "MLP-GEMM-2 fwd"),
                              (H, 3 * H // world, True, "qkv dgrad"), (H, 4 * H // world, True, "MLP-GEMM-1 dgrad")]:
        x = torch.randn(M, k, device=dev, dtype=dt)
        w = torch.randn((k, n) if b_mn else (n, k), device=dev, dtype=dt) * 0.05
        out = torch.empty(M, n, device=dev, dtype=dt)
        rs = torch.empty(M // world, n, device=dev, dtype=dt)
        gemm_us = timeit(lambda: ops.gemm(x, w, b_mn=b_mn, out=out))

        def ar_base():
            ops.gemm(x, w, b_mn=b_mn, out=out)
            dist.all_reduce(out)

        def rs_base():
            ops.gemm(x, w, b_mn=b_mn, out=out)
            dist.reduce_scatter_tensor(rs, out)

        # all-reduce: partial tiles out + reduced tiles out, each (W-1)/W of the output, per GPU and direction
        report("gemm_allreduce", tag, n, k, timeit(lambda: be.gemm_all_reduce(x, w, b_mn=b_mn)), timeit(ar_base),
               gemm_us, 2 * frac * M * n * esz)
        report("gemm_reduce_scatter", tag, n, k, timeit(lambda: be.gemm_reduce_scatter(x, w, b_mn=b_mn)),
               timeit(rs_base), gemm_us, frac * M * n * esz)
    for (n, k, tag) in [(3 * H // world, H, "qkv fwd"), (4 * H // world, H, "MLP-GEMM-1 fwd")]:
        w = torch.randn(n, k, device=dev, dtype=dt) * 0.05
        out = torch.empty(M, n, device=dev, dtype=dt)
        gathered = torch.empty(M, k, device=dev, dtype=dt)
        block = torch.randn(M // world, k, device=dev, dtype=dt)
        full, mine = be.gather_buffer(M, k)
        mine.copy_(block)

        def fused():
            # the producing kernel would write `mine` directly; the block is already in place here
            be.gemm_all_gather(full, w, out=out)

        def base():
            dist.all_gather_into_tensor(gathered, block)
            ops.gemm(gathered, w, out=out)

        report("allgather_gemm", tag, n, k, timeit(fused), timeit(base), timeit(lambda: ops.gemm(gathered, w, out=out)),
               frac * M * k * esz)
    native.check_status()
    be.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
