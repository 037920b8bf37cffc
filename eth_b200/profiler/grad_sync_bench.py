"""Block-wise gradient all-reduce micro-benchmark: bucket-size sweep on one transformer layer's
gradients.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29535 -m eth_b200.profiler.grad_sync_bench [--hidden 4096] [--dtype bf16]

The gradients of one layer (12 h^2 + 13 h elements; GPT-6.7B: 201 M) are reduced over all ranks
  * tensor-wise with NCCL (one all-reduce per parameter tensor, the reference's `tensor` mode),
    alone and followed by torch's fused AdamW on fp32 master weights,
  * bucketed with NCCL (`block` mode) for bucket sizes 1..256 MiB,
  * bucketed with the one-shot peer-memory kernel (`peer_allreduce`: every rank reads all peers),
  * bucketed with the two-shot in-place peer-memory kernel (`peer_reduce_pieces`: no pack, no unpack,
    waiting done by one-warp flag kernels), alone, followed by this library's fused AdamW (unscale,
    clip, update, 16-bit refresh in one pass), and started on a side stream while the GEMMs of one
    layer's backward run on the main stream: `exposed_ms` is what that adds to the backward alone,
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

    # optimizer state of the layer: fp32 master + moments, 16-bit weights
    from eth_b200.ops import functional  # noqa: F401  (loads the native library)
    flags2 = SymmetricBuffer(64 * 4, ranks, rank, None, dev)
    epoch2 = [0]
    side = torch.cuda.Stream(device=dev)
    param16 = torch.zeros(total, device=dev, dtype=dt if dt != torch.float32 else torch.bfloat16)
    master = torch.randn(total, device=dev) * 0.02
    m1, m2 = torch.zeros_like(master), torch.zeros_like(master)
    ctrl = torch.zeros(4, device=dev)
    ctrl[2] = 1.0 / 4096.0
    torch_master = torch.nn.Parameter(master.clone())
    torch_opt = torch.optim.AdamW([torch_master], lr=1.5e-4, weight_decay=0.01, fused=True)

    def adam_ours():
        ctrl[:2].zero_()
        native.lib().grad_norm_sq(mine, 1.0, ctrl)
        native.lib().fused_adam(param16, master, mine, m1, m2, ctrl, 1.5e-4, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, 1.0, True, True)

    def adam_torch():
        torch_master.grad = grads.float().mul_(1.0 / 4096.0)   # cast + unscale pass of the reference optimizer
        torch.nn.utils.clip_grad_norm_([torch_master], 1.0)
        torch_opt.step()
        param16.copy_(torch_master.detach())

    # GEMMs of one layer's backward (data and weight gradients of the four linears), 4096 tokens
    tokens = 4096
    xs = {n: torch.randn(tokens, n, device=dev, dtype=torch.bfloat16) * 0.1 for n in (h, 3 * h, 4 * h)}
    ws = [(torch.randn(3 * h, h, device=dev, dtype=torch.bfloat16) * 0.02, 3 * h, h),
          (torch.randn(h, h, device=dev, dtype=torch.bfloat16) * 0.02, h, h),
          (torch.randn(4 * h, h, device=dev, dtype=torch.bfloat16) * 0.02, 4 * h, h),
          (torch.randn(h, 4 * h, device=dev, dtype=torch.bfloat16) * 0.02, h, 4 * h)]
    wg = [torch.zeros(o, i, device=dev, dtype=torch.float32) for _, o, i in ws]

    def backward_standin():
        for (w, o, i), g in zip(ws, wg):
            functional.gemm(xs[o], w, b_mn=True)                                   # dX = dY W
            functional.gemm(xs[o], xs[i], a_mn=True, b_mn=True, out=g, accumulate=True)   # dW += dY^T X

    t_bwd = timeit(backward_standin)

    def tensor_wise_adam():
        tensor_wise()
        adam_torch()

    emit(mode="tensor-wise NCCL", tensors=len(shapes), ms=round(timeit(tensor_wise), 3),
         plus_torch_adamw_ms=round(timeit(tensor_wise_adam), 3), backward_alone_ms=round(t_bwd, 3),
         exposed_ms=round(timeit(tensor_wise), 3))
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

        tables = [torch.tensor([[o, 1, (n + 7) // 8 * 8, (n + 7) // 8 * 8]], dtype=torch.int64, device=dev) for o, n in cuts]

        def two_shot(wait=True):
            st = native.status(dev)
            for tab in tables:
                epoch2[0] += 1
                native.lib().peer_flags(flags2.ptrs, rank, epoch2[0], 0, 0, st)
                native.lib().peer_reduce_pieces(sym.ptrs, flags2.ptrs, rank, epoch2[0], tab, code, 1.0 / world)   # mean: values stay bounded over repeats
            if wait:
                native.lib().peer_flags(flags2.ptrs, rank, epoch2[0], -1, 8, st)

        def two_shot_adam():
            two_shot()
            adam_ours()

        def overlapped():
            # one layer's backward on the main stream; the buckets reduce on a side stream meanwhile
            ready = torch.cuda.Event()
            ready.record()
            side.wait_event(ready)
            with torch.cuda.stream(side):
                two_shot(wait=False)
            backward_standin()
            torch.cuda.current_stream().wait_stream(side)
            native.lib().peer_flags(flags2.ptrs, rank, epoch2[0], -1, 8, native.status(dev))

        t_n, t_p, t_2 = timeit(nccl_buckets), timeit(peer_buckets), timeit(two_shot)
        t_2a, t_ov = timeit(two_shot_adam), timeit(overlapped)
        emit(mode="block", bucket_mb=mb, buckets=len(cuts), nccl_ms=round(t_n, 3), one_shot_ms=round(t_p, 3),
             two_shot_ms=round(t_2, 3), two_shot_plus_fused_adam_ms=round(t_2a, 3),
             two_shot_busbw_gbs=round(2 * (world - 1) / world * total * esz / (t_2 * 1e-3) / 1e9, 1),
             backward_alone_ms=round(t_bwd, 3), overlapped_total_ms=round(t_ov, 3),
             exposed_ms=round(max(0.0, t_ov - t_bwd), 3))
    native.check_status()
    for b in (sym, flags, flags2):
        b.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
