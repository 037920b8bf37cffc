"""CUDA-event micro-benchmarks of single kernels, reported against the measured roofline.

    python -m eth_b200.profiler.kernel_bench gemm --m 8192 --n 8192 --k 8192 [--dtype bf16]
    python -m eth_b200.profiler.kernel_bench attn --batch 4 --seq 2048 --heads 16 --dim 128
    python -m eth_b200.profiler.kernel_bench ln --rows 8192 --hidden 2048

Timing rules: warm-up launches first, L2 flushed (a 256 MiB buffer is overwritten) before every
timed launch, CUDA events on the launching stream, median of the repeats.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def time_fn(fn, warmup=5, repeat=20, flush=True):
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeat):
        if flush_buf is not None:
            flush_buf.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times), min(times)


def main(argv=None):
    from eth_b200 import ops
    from eth_b200.ops import native

    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["gemm", "attn", "ln", "gemm_sweep", "elementwise"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--repeat", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--compare", action="store_true", help="also time the torch library op")
    args = ap.parse_args(argv)
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    hbm, tflops_peak, src = _peaks()
    out = []

    def gemm_case(M, N, K, a_mn, b_mn):
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=dt)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=dt)
        d = torch.empty(M, N, device="cuda", dtype=dt)
        med, best = time_fn(lambda: ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=d), args.warmup, args.repeat)
        native.check_status()
        fl = 2.0 * M * N * K
        rec = {"kernel": "gemm_tcgen05", "M": M, "N": N, "K": K, "a_mn": a_mn, "b_mn": b_mn,
               "ms_median": med, "ms_best": best, "tflops": fl / med / 1e9,
               "frac_of_%s_bf16_peak" % src: fl / med / 1e9 / tflops_peak}
        if args.compare:
            am = a.t() if a_mn else a
            bm = b if b_mn else b.t()
            med2, _ = time_fn(lambda: torch.matmul(am, bm, out=d), args.warmup, args.repeat)
            rec["torch_matmul_ms"] = med2
            rec["torch_matmul_tflops"] = fl / med2 / 1e9
        return rec

    if args.kind == "gemm":
        out.append(gemm_case(args.m, args.n, args.k, args.a_mn, args.b_mn))
    elif args.kind == "gemm_sweep":
        for (M, N, K, am, bm) in [(8192, 8192, 8192, False, False), (8192, 6144, 2048, False, False),
                                  (8192, 2048, 2048, False, False), (8192, 8192, 2048, False, False),
                                  (8192, 2048, 8192, False, False), (8192, 2048, 6144, False, True),
                                  (6144, 2048, 8192, True, True), (8192, 50432, 2048, False, False),
                                  (8192, 12288, 4096, False, False), (8192, 4096, 16384, False, False)]:
            out.append(gemm_case(M, N, K, am, bm))
    elif args.kind == "attn":
        B, S, H, D = args.batch, args.seq, args.heads, args.dim
        qkv = torch.randn(B, S, H, 3, D, device="cuda", dtype=dt)
        q, k, v = qkv[:, :, :, 0], qkv[:, :, :, 1], qkv[:, :, :, 2]
        fl = 4.0 * B * H * S * S * D / 2  # causal
        if not args.bwd:
            med, best = time_fn(lambda: ops.flash_attention(q, k, v), args.warmup, args.repeat)
            native.check_status()
            rec = {"kernel": "attention_fwd", "B": B, "S": S, "H": H, "D": D, "ms_median": med,
                   "tflops": fl / med / 1e9, "frac_of_%s_bf16_peak" % src: fl / med / 1e9 / tflops_peak}
            if args.compare:
                qt, kt, vt = (t.permute(0, 2, 1, 3) for t in (q, k, v))
                med2, _ = time_fn(lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True),
                                  args.warmup, args.repeat)
                rec["torch_sdpa_ms"] = med2
        else:
            qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
            o = ops.flash_attention(qg, kg, vg)
            do = torch.randn_like(o)
            med, best = time_fn(lambda: torch.autograd.grad(o, (qg, kg, vg), do, retain_graph=True),
                                args.warmup, args.repeat)
            native.check_status()
            rec = {"kernel": "attention_bwd", "B": B, "S": S, "H": H, "D": D, "ms_median": med,
                   "tflops": 2.5 * fl / med / 1e9}
            if args.compare:   # the library backward (cuDNN / flash kernels behind torch SDPA) on the same tensors
                qt, kt, vt = (t.detach().permute(0, 2, 1, 3).clone().requires_grad_(True) for t in (q, k, v))
                ot = torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
                dot = torch.randn_like(ot)
                med2, _ = time_fn(lambda: torch.autograd.grad(ot, (qt, kt, vt), dot, retain_graph=True),
                                  args.warmup, args.repeat)
                rec["torch_sdpa_bwd_ms"] = med2
        out.append(rec)
    elif args.kind == "ln":
        x = torch.randn(args.rows, args.hidden, device="cuda", dtype=dt)
        g = torch.ones(args.hidden, device="cuda", dtype=dt)
        b = torch.zeros(args.hidden, device="cuda", dtype=dt)
        med, best = time_fn(lambda: ops.layer_norm(x, g, b), args.warmup, args.repeat)
        byts = 2.0 * x.numel() * x.element_size()
        out.append({"kernel": "ln_fwd", "rows": args.rows, "hidden": args.hidden, "ms_median": med,
                    "gbs": byts / med / 1e6, "frac_of_%s_hbm" % src: byts / med / 1e6 / hbm})
    elif args.kind == "elementwise":
        # the memory-bound kernels of a transformer layer on [rows, hidden]; bytes = algorithmic traffic
        from eth_b200.ops import raw
        rows, h = args.rows, args.hidden
        x = torch.randn(rows, h, device="cuda", dtype=dt)
        g = torch.ones(h, device="cuda", dtype=dt)
        b = torch.zeros(h, device="cuda", dtype=dt)
        g.main_grad = torch.zeros(h, device="cuda")
        b.main_grad = torch.zeros(h, device="cuda")
        _, mean, rstd = raw.ln_fwd(x, g, b, 1e-5)
        dy, res = torch.randn_like(x), torch.randn_like(x)
        bias = torch.zeros(h, device="cuda", dtype=dt)
        nb = x.numel() * x.element_size()
        cases = [("ln_fwd", lambda: raw.ln_fwd(x, g, b, 1e-5), 2 * nb),
                 ("ln_bwd", lambda: raw.ln_bwd(dy, x, g, b, mean, rstd), 3 * nb),
                 ("ln_bwd + residual gradient", lambda: raw.ln_bwd(dy, x, g, b, mean, rstd, residual_grad=res), 4 * nb),
                 ("bias_dropout_add_fwd", lambda: raw.bias_dropout_add_fwd(x, bias, res, 0.1, 1, 2), 3 * nb),
                 ("dropout_bwd + bias-gradient column sums", lambda: raw.dropout_bwd_colsum(dy, 0.1, 1, 2), 2 * nb)]
        # the same two backward kernels as the training step runs them on all but the last micro-batch:
        # partial column sums stay in the op's slabs, no second launch
        bias.main_grad = torch.zeros(h, device="cuda")
        ln_slabs, drop_slabs = raw.ColumnSumSlabs(), raw.ColumnSumSlabs()
        cases += [("ln_bwd + residual gradient, column sums deferred",
                   lambda: raw.ln_bwd(dy, x, g, b, mean, rstd, residual_grad=res, slabs=ln_slabs,
                                      ws_mode=raw.WS_ACCUMULATE), 4 * nb),
                  ("dropout_bwd, bias-gradient column sums deferred",
                   lambda: raw.dropout_bwd_colsum_into(dy, 0.1, 1, 2, bias.main_grad, drop_slabs, raw.WS_ACCUMULATE),
                   2 * nb)]
        for name, fn, byts in cases:
            med, best = time_fn(fn, args.warmup, args.repeat)
            out.append({"kernel": name, "rows": rows, "hidden": h, "ms_median": med, "gbs": byts / med / 1e6,
                        "frac_of_%s_hbm" % src: byts / med / 1e6 / hbm})
    for rec in out:
        print(json.dumps(rec))
    return out


if __name__ == "__main__":
    main()
