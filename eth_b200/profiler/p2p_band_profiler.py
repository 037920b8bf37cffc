"""Point-to-point bandwidth profiler (2 ranks): for sizes 2^0..2^10 MB of fp16, 20 warm-up and 50
timed transfers in each direction; appends three CSV rows -- sizes (MB), send GB/s, recv GB/s
(reference: eth/profiler/p2p_band_profiler.py:20-95; the `_i` twin uses isend/irecv, selected here
with P2P_NONBLOCKING=1). Environment: FILE_NAME, NNODES, GPUS_PER_NODE, NODE_RANK, MASTER_ADDR,
MASTER_PORT. Timing: CUDA events, not host wall-clock.
"""
from __future__ import annotations

import csv
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

SIZES_MB = [2 ** i for i in range(11)]
WARMUP, REPEAT = 20, 50


def _transfer(x, peer, send: bool, nonblocking: bool):
    if nonblocking:
        (dist.isend(x, peer) if send else dist.irecv(x, peer)).wait()
    elif send:
        dist.send(x, peer)
    else:
        dist.recv(x, peer)


def run(rank: int, world: int, file_name: str, nonblocking: bool):
    device = torch.device("cuda", torch.cuda.current_device())
    peer = 1 - rank
    send_bw, recv_bw = [], []
    for size in SIZES_MB:
        x = torch.ones(size * 1024 * 1024 // 2, dtype=torch.float16, device=device)
        for direction in (0, 1):      # 0: rank 0 sends, 1: rank 1 sends
            sender = rank == direction
            for _ in range(WARMUP):
                _transfer(x, peer, sender, nonblocking)
            torch.cuda.synchronize()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(REPEAT):
                _transfer(x, peer, sender, nonblocking)
            e.record()
            e.synchronize()
            gbs = size / 1024.0 * REPEAT / (s.elapsed_time(e) / 1e3)
            if rank == 0:
                (send_bw if direction == 0 else recv_bw).append(gbs)
    if rank == 0:
        with open(file_name, "a", newline="") as f:
            w = csv.writer(f)
            w.writerow(SIZES_MB)
            w.writerow([f"{b:.4f}" for b in send_bw])
            w.writerow([f"{b:.4f}" for b in recv_bw])


def init_process(local_rank: int, nnodes: int, gpus_per_node: int, node_rank: int, file_name: str):
    rank = node_rank * gpus_per_node + local_rank
    world = nnodes * gpus_per_node
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
    run(rank, world, file_name, os.environ.get("P2P_NONBLOCKING", "0") == "1")
    dist.destroy_process_group()


def main():
    file_name = os.environ.get("FILE_NAME", "p2p_intra_node.csv")
    nnodes = int(os.environ.get("NNODES", "1"))
    gpn = int(os.environ.get("GPUS_PER_NODE", "2"))
    node_rank = int(os.environ.get("NODE_RANK", "0"))
    if nnodes * gpn != 2:
        raise SystemExit("the P2P profiler runs on exactly two ranks")
    if os.path.exists(file_name) and node_rank == 0:
        os.remove(file_name)
    mp.spawn(init_process, args=(nnodes, gpn, node_rank, file_name), nprocs=gpn, join=True)


if __name__ == "__main__":
    main()
