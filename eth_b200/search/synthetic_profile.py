"""Deterministic synthetic profile directory (for CPU-only search runs and tests).

Per-op forward/backward times ~ U(1, 3) ms per layer scaled by micro-batch and 1/TP, collectives
and P2P follow latency = alpha + bytes / beta with alpha = 10 us, beta = 20 GB/s by default, and
memory columns follow the GPT shapes of the requested size.

    python -m eth_b200.search.synthetic_profile --output prof --model-size 1_3B --hardware example-gpu --tp-sizes 1,2,4
"""
from __future__ import annotations

import argparse
import csv
import os
import random

from ..contract.config import FIRST_OP, GPT_SIZES, LAYER_OPS, TAIL_OPS
from ..profiler.profile_metadata import write_metadata
from .profile_db import COLLECTIVES, OP_HEADER


def _shares():
    # rough share of a layer's time per op (GEMMs dominate)
    return {"enc-1st-layernorm": 0.02, "enc-attention-qkv": 0.18, "enc-flash-attention": 0.12,
            "enc-attention-dense": 0.07, "enc-post-attention-dropout": 0.02, "enc-2nd-layernorm": 0.02,
            "enc-MLP-GEMM-1": 0.26, "enc-MLP-gelu": 0.02, "enc-MLP-GEMM-2": 0.27, "enc-post-MLP-dropout": 0.02}


def generate(output, model_size="1_3B", hardware="example-gpu", tp_sizes=(1, 2, 4), mbs_list=(1, 2, 4, 8), seed=0,
             alpha_us=10.0, beta_gbs=20.0, vocab=51200, status="complete", slowdown=1.0):
    m = GPT_SIZES[model_size]
    h, s = m["hidden_size"], m["seq_length"]
    rng = random.Random(seed)
    layer_fwd_ms = rng.uniform(1.0, 3.0) * slowdown     # one layer, mbs 1, TP 1 (`slowdown` > 1: a slower GPU type)
    layer_bwd_ms = rng.uniform(1.0, 3.0) * 2 * slowdown
    os.makedirs(output, exist_ok=True)
    mb = 1.0 / (1024 * 1024)
    sizes = set()
    for mbs in mbs_list:
        for tp in tp_sizes:
            for algo in (0, 1):
                rows = []
                act = mbs * s * h * 2 * mb
                def row(name, f_ms, b_ms, inp, out, w, a):
                    sizes.update([round(inp, 4), round(out, 4)])
                    rows.append([name, f"{f_ms * 1e3:.3f}", f"{b_ms * 1e3:.3f}", f"{inp:.4f}", f"{out:.4f}", f"{w:.4f}",
                                 f"{a:.4f}", f"{out:.4f}", f"{out * 2:.4f}"])
                row(FIRST_OP, 0.05 * mbs, 0.08 * mbs, mbs * s * 8 * mb, act, (vocab * h / tp + s * h) * 2 * mb, act)
                weights = {"enc-attention-qkv": 3 * h * h / tp, "enc-attention-dense": h * h / tp,
                           "enc-MLP-GEMM-1": 4 * h * h / tp, "enc-MLP-GEMM-2": 4 * h * h / tp}
                outs = {"enc-attention-qkv": 3 * act / tp, "enc-flash-attention": act / tp, "enc-MLP-GEMM-1": 4 * act / tp,
                        "enc-MLP-gelu": 4 * act / tp}
                ins = {"enc-flash-attention": 3 * act / tp, "enc-attention-dense": act / tp, "enc-MLP-gelu": 4 * act / tp,
                       "enc-MLP-GEMM-2": 4 * act / tp}
                for name in LAYER_OPS:
                    share = _shares()[name]
                    scale = mbs / (tp if name not in ("enc-1st-layernorm", "enc-2nd-layernorm", "enc-post-attention-dropout",
                                                        "enc-post-MLP-dropout") else 1)
                    jitter = 1.0 + 0.02 * algo
                    row(name, layer_fwd_ms * share * scale * jitter, layer_bwd_ms * share * scale * jitter,
                        ins.get(name, act), outs.get(name, act), weights.get(name, 2 * h if "layernorm" in name else 0) * 2 * mb,
                        outs.get(name, act))
                row(TAIL_OPS[0], 0.02 * mbs, 0.04 * mbs, act, act, 2 * h * 2 * mb, act)
                row(TAIL_OPS[1], 0.3 * mbs / tp, 0.6 * mbs / tp, act, mbs * s * 4 * mb, 0.0, mbs * s * vocab / tp * 2 * mb)
                with open(os.path.join(output, f"gpt_{model_size}_mbs{mbs}_tp{tp}_algo{algo}.csv"), "w", newline="") as f:
                    w = csv.writer(f)
                    w.writerow(OP_HEADER)
                    w.writerows(rows)
    size_list = sorted(x for x in sizes if x > 0)
    for tp in tp_sizes:
        if tp == 1:
            continue
        for prim in COLLECTIVES:
            with open(os.path.join(output, f"prim_gpt_{model_size}_{prim}_{tp}gpus.csv"), "w", newline="") as f:
                w = csv.writer(f)
                w.writerow(["data_size(MB)", "time(ms)"])
                for sz in size_list:
                    factor = 2.0 * (tp - 1) / tp if prim == "all_reduce" else (tp - 1) / tp
                    w.writerow([sz, f"{alpha_us / 1e3 + sz / 1024.0 / beta_gbs * 1e3 * factor:.5f}"])
    p2p_sizes = [2 ** i for i in range(11)]
    bw = [sz / 1024.0 / (alpha_us * 1e-6 + sz / 1024.0 / beta_gbs) for sz in p2p_sizes]
    with open(os.path.join(output, "p2p_intra_node.csv"), "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(p2p_sizes)
        w.writerow([f"{b:.4f}" for b in bw])
        w.writerow([f"{b:.4f}" for b in bw])
    write_metadata(output, status, model_size, hardware, tp_sizes, 1, max(tp_sizes), 0)
    return output


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--output", required=True)
    ap.add_argument("--model-size", default="1_3B")
    ap.add_argument("--hardware", default="example-gpu")
    ap.add_argument("--tp-sizes", default="1,2,4")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    generate(a.output, a.model_size, a.hardware, [int(t) for t in a.tp_sizes.split(",")], seed=a.seed)


if __name__ == "__main__":
    main()
