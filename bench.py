"""Headline benchmark: GPT training throughput (tokens/s, whole job) on N GPUs of one node.

    python bench.py --gpus 1 --steps 4 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 4 --warmup 3
    python bench.py --impl reference --gpus 1 ...      (the unmodified reference, if installed)

Model and layout follow the GPT-1.3B fp16 training config (24 layers, hidden 2048, 16 heads,
seq 2048, vocab 50257, micro-batch 4 per data-parallel replica, block-wise gradient sync with 32 MiB buckets):
    8 GPUs: PP2 x TP2 x DP2, global batch 512 (the layout the benchmark definition fixes)
    4 GPUs: DP4, global batch 256      2 GPUs: DP2, global batch 128      1 GPU: global batch 64
so the work per GPU is constant (weak scaling). GPT-1.3B fits one B200, and on the measured profile the
configuration search prefers replicas over tensor parallelism for 2 and 4 GPUs, so those sizes use it. Data is synthetic (closed-form token ids), weights
are random-init.

Two numbers are measured, both with CUDA events around exactly K steps, bracketed by a barrier and
a device synchronize, max over ranks:
  value : steps whose batches are generated on the device (kernel-side throughput);
  e2e   : the same steps through the public `TrainEngine.train_step()` API with every step's
          token ids / labels / loss mask built on the host, copied from pinned memory, and the
          step's loss read back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODEL = dict(model_size="1_3B", num_layers=24, hidden_size=2048, num_attention_heads=16, seq_length=2048,
             max_position_embeddings=2048)
VOCAB = 50257
MICRO_BATCH = 4
SAMPLES_PER_GPU = 64
LAYOUTS = {1: (1, 1, 1), 2: (1, 1, 2), 4: (1, 1, 4), 8: (2, 2, 2)}  # N -> (pp, tp, dp)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        return self.summary(self.lines)

    @staticmethod
    def summary(lines):
        """Median SM clock, highest maximum clock and the throttle reasons seen in the sampled lines."""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_config(n_gpus: int):
    from eth_b200.contract.config import uniform_config
    pp, tp, dp = LAYOUTS[n_gpus]
    gbs = SAMPLES_PER_GPU * n_gpus
    # a pipe's micro_batch_size spans its DP replicas; every replica runs MICRO_BATCH samples per micro-batch
    return uniform_config(MODEL, pp=pp, tp=tp, dp=dp, gbs=gbs, mbs=MICRO_BATCH * dp), (pp, tp, dp), gbs


def run_ours(opts):
    import torch
    import torch.distributed as dist
    from eth_b200.ops import native
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != opts.gpus:
        raise SystemExit(f"--gpus {opts.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    config, (pp, tp, dp), gbs = build_config(opts.gpus)
    argv = ["--fp16", "--loss-scale", "4096", "--hidden-dropout", "0.1", "--grad-sync-mode", "block",
            "--grad-sync-bucket-size-mb", "32", "--train-iters", str(opts.steps + opts.warmup),
            "--vocab-size", str(VOCAB)]
    if opts.bf16:
        argv = ["--bf16"] + argv[3:]
    argv += opts.engine_args.split()
    args = parse_args(argv, config=config, rank=rank, world_size=world, local_rank=local_rank)
    engine = TrainEngine(args)

    def barrier_sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(k, e2e):
        losses = []
        barrier_sync()
        l0 = native.launch_count()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(k):
            engine.train_step()
            if e2e:
                losses.append(engine.reduced_loss())   # device -> host read of the step's result
        e.record()
        barrier_sync()
        ms = s.elapsed_time(e)
        t = torch.tensor([ms], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), native.launch_count() - l0, losses

    # A bounded device wait that expired during warm-up (ranks of a peer group that started more than
    # the wait limit apart) is reported in the JSON line and cleared: the engine raises on every rank
    # in the same step (the fault mark travels with the overflow flag), the update of that step was
    # skipped everywhere, and the ranks go on together. One inside the timed region invalidates the
    # measurement and ends the run.
    warmup_status = None
    barrier_sync()          # all ranks begin their first step together
    for _ in range(opts.warmup):
        try:
            engine.train_step()
        except RuntimeError as err:
            if "bounded device wait" not in str(err):
                raise
            warmup_status = str(err)
            try:
                native.check_status()      # reads and clears this rank's status word
            except RuntimeError:
                pass
            barrier_sync()
    try:
        native.check_status()
    except RuntimeError as err:
        warmup_status = str(err)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms, launches, _ = timed(opts.steps, e2e=False)
    clocks = sampler.stop() if sampler else None
    # exposed gradient-sync time: what the main stream spends reducing gradients after the last
    # backward of an iteration (CUDA events inside the engine), mean over the timed steps, max over ranks
    gs = torch.tensor([engine.exposed_grad_sync_ms(last=opts.steps)], device="cuda")
    if world > 1:
        dist.all_reduce(gs, op=dist.ReduceOp.MAX)
    exposed_ms = float(gs.item())
    native.check_status()
    tokens = gbs * MODEL["seq_length"] * opts.steps
    value = tokens / (ms / 1e3)

    # end-to-end arm: host-built batches from pinned memory + loss read-back every step
    from eth_b200.data.provider import SyntheticHostProvider
    provider = SyntheticHostProvider(VOCAB)   # what --host-data selects in the training entry point
    engine.data_provider = provider
    engine.train_step()
    provider.reset_counter()
    ms_e2e, _, losses = timed(opts.steps, e2e=True)
    e2e_value = tokens / (ms_e2e / 1e3)
    native.check_status()
    if rank == 0:
        out = {
            "metric": "GPT training throughput (tokens/s, device-timed, max over ranks)",
            "value": value, "unit": "tokens/s", "n_gpus": opts.gpus, "steps": opts.steps, "warmup": opts.warmup,
            "ms_per_step": ms / opts.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if opts.bf16 else "fp16", "data": "synthetic token ids, random-init weights",
            "impl": "eth_b200",
            "config": {"model": "GPT-1.3B (24 layers, hidden 2048, 16 heads)", "global_batch": gbs,
                       "seq_len": MODEL["seq_length"], "micro_batch": MICRO_BATCH, "pipeline_micro_batch": MICRO_BATCH * dp,
                       "parallelism": f"pp{pp}tp{tp}dp{dp}", "grad_sync": "block, 32 MiB buckets", **({"engine_args": opts.engine_args} if opts.engine_args else {}),
                       "l2": "inputs larger than L2 (each step streams several GB of weights and activations)"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / opts.steps,
                    "h2d_bytes_per_step": provider.h2d_bytes // opts.steps, "d2h_bytes_per_step": 8,
                    "final_loss": losses[-1] if losses else None},
            "gpu_launches": launches,
            "exposed_grad_sync_ms_per_step": exposed_ms,
        }
        if warmup_status:
            out["warmup_status"] = warmup_status
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_reference(opts):
    from baseline.reference_arm import run as run_ref
    run_ref(opts, MODEL, LAYOUTS, SAMPLES_PER_GPU, MICRO_BATCH, VOCAB, clock_sampler_cls=ClockSampler)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bf16", action="store_true", help="bf16 instead of the config's fp16")
    ap.add_argument("--layout", default=None,
                    help="pp,tp,dp to use instead of the default layout of --gpus (same model, batch per GPU and "
                         "metric; for studying a layout, e.g. 2,2,1 on four GPUs)")
    ap.add_argument("--engine-args", default="",
                    help="extra engine flags for studying a variant, e.g. '--p2p-backend nccl' (own arm only)")
    opts = ap.parse_args()
    if opts.layout:
        pp, tp, dp = (int(v) for v in opts.layout.split(","))
        if pp * tp * dp != opts.gpus:
            raise SystemExit("--layout must multiply to --gpus")
        LAYOUTS[opts.gpus] = (pp, tp, dp)
    if opts.gpus not in LAYOUTS:
        raise SystemExit(f"--gpus must be one of {sorted(LAYOUTS)}")
    if opts.impl == "reference":
        run_reference(opts)
    else:
        run_ours(opts)


if __name__ == "__main__":
    main()
