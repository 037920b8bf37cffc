"""Block-wise gradient all-reduce micro-benchmark: bucket-size sweep on one transformer layer's
gradients.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29535 -m eth_b200.profiler.grad_sync_bench [--hidden 4096] [--dtype bf16]

The gradients of one layer (12 h^2 + 13 h elements; GPT-6.7B: 201 M) are reduced over all ranks
  * tensor-wise with NCCL (one all-reduce per parameter tensor, the reference's `tensor` mode),
  * bucketed with NCCL (`block` mode) for bucket sizes 1..256 MiB,
  * bucketed with the one-shot peer-memory kernel (`peer_allreduce`, fused normalisation scale),
timed with CUDA events after warm-up, maximum over ranks. One JSON line per case.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    from eth_b200.ops import native
    from eth_b200.parallel.peer_memory import SymmetricBuffer

    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--repeat", type=int, default=10)
    ap.add_argument("--sizes-mb", default="1,2,4,8,16,32,64,128,256")
    a = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dt]
    h = a.hidden
    shapes = [3 * h * h, 3 * h, h * h, h, 4 * h * h, 4 * h, 4 * h * h, h, h, h, h, h]   # weights and biases of a layer
    total = sum(shapes)
    esz = torch.empty((), dtype=dt).element_size()
    grads = torch.randn(total, device=dev, dtype=torch.float32).to(dt)
    ranks = tuple(range(world))
    sym = SymmetricBuffer(total * esz, ranks, rank, None, dev)
    flags = SymmetricBuffer(64 * 4, ranks, rank, None, dev)
    mine = sym.tensor((total,), dt)
    out = torch.empty(total, device=dev, dtype=dt)
    epoch = [0]

    def timeit(fn):
        for _ in range(3):
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
        return t.item()

    def emit(**kw):
        if rank == 0:
            print(json.dumps(dict(kw, world=world, dtype=a.dtype, layer_mbytes=round(total * esz / 2 ** 20, 1))), flush=True)

    def tensor_wise():
        off = 0
        for n in shapes:
            dist.all_reduce(grads[off:off + n])
            off += n

    emit(mode="tensor-wise NCCL", tensors=len(shapes), ms=round(timeit(tensor_wise), 3))
    for mb in [int(x) for x in a.sizes_mb.split(",")]:
        per = mb * 2 ** 20 // esz
        cuts = [(o, min(per, total - o)) for o in range(0, total, per)]

        def nccl_buckets():
            for o, n in cuts:
                dist.all_reduce(grads[o:o + n])

        def peer_buckets():
            mine.copy_(grads)                       # stands for the pack pass of the executor
            for o, n in cuts:
                epoch[0] += 1
                native.lib().peer_allreduce([p + o * esz for p in sym.ptrs], flags.ptrs, rank, epoch[0], n, code, 1.0,
                                            out[o:o + n], None, 0.0, native.status(dev))

        t_n, t_p = timeit(nccl_buckets), timeit(peer_buckets)
        emit(mode="block", bucket_mb=mb, buckets=len(cuts), nccl_ms=round(t_n, 3), peer_kernel_ms=round(t_p, 3),
             peer_busbw_gbs=round(2 * (world - 1) / world * total * esz / (t_p * 1e-3) / 1e9, 1))
    native.check_status()
    for b in (sym, flags):
        b.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
