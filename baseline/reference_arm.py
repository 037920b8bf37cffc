"""Reference arm of the benchmark: the unmodified YuMJie/ETH runtime, timed in this process.

Where the code comes from
    `baseline/_ref/` is a byte-identical copy of the reference source tree (the pip route stops in
    metadata generation: the tree has no packaging metadata and setuptools' flat-layout discovery
    sees three top-level packages). Nothing below writes into that copy except the reference's own
    JIT build directories (`megatron/fused_kernels/build`, `megatron/data/helpers*.so`).

What runs
    The reference's training program, `eth/runtime/pretrain_gpt.py` (its `__main__` block calls
    `pretrain(train_valid_test_datasets_provider, model_provider, forward_step, ...)`,
    pretrain_gpt.py:157-165), with the argument list its launcher passes
    (scripts/train_gpt.sh:286-309) for the same model, layout, batch sizes, precision and
    block-wise gradient sync with 32 MiB buckets as the other arm. The launcher script itself is
    bypassed because it insists on CUDA 12.4 and a populated Apex checkout
    (scripts/train_gpt.sh:226-235,270-273).

Shims, all outside the reference tree
    * `baseline/shims/apex`: importable stand-in that reports the fused extensions as missing, so
      the reference's own fallbacks (torch AdamW, PyTorch norm / scale) run.
    * `torch.utils.cpp_extension.load` is wrapped for the duration of the run
      (`baseline/reference_build.py`): it appends `-gencode arch=compute_100,code=sm_100` to
      `extra_cuda_cflags` (the reference lists only sm_70 / sm_80, fused_kernels/__init__.py:36-54),
      reuses an ahead-of-time build of the same sources when there is one, and registers the
      extension in `sys.modules` so the reference's by-name imports find it.
    * `PROFILING` environment variable: the reference's timers synchronise the device on every
      start/stop when it is 1, its default (global_vars.py:43,203-220). Both variants can be
      recorded; `ETHB_REF_PROFILING` selects one (default 0, the faster).

Timing
    `megatron.training.train_step` is wrapped (module attribute, no file is edited): after the
    warm-up calls a barrier and a device synchronise bracket the timed calls; CUDA events around
    every timed `train_step` give the device-side number, and one event pair spanning the timed
    iterations including the reference's per-iteration logging (which reads loss, loss scale and
    gradient norm back to the host) gives the end-to-end number. Maximum over ranks.

Any exception raised by the reference under these shims is reported as
`{"impl": "reference", "unavailable": "<file:line: message>"}` with exit status 0.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile
import threading
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")
REF_RUNTIME = os.path.join(REF_ROOT, "eth", "runtime")
SHIMS = os.path.join(HERE, "shims")


def _first_reference_frame(exc: BaseException) -> str:
    """`path:line` of the innermost frame that lies in the reference tree (or the innermost frame)."""
    frames = traceback.extract_tb(exc.__traceback__)
    inside = [f for f in frames if os.path.realpath(f.filename).startswith(os.path.realpath(REF_ROOT))]
    f = (inside or frames or [None])[-1]
    if f is None:
        return "?"
    name = os.path.relpath(os.path.realpath(f.filename), os.path.realpath(REF_ROOT)) if inside else f.filename
    return f"{name}:{f.lineno}"


def write_config(path: str, model, layout, gbs: int, micro_batch: int) -> None:
    """The benchmark layout as a `gpt_config.json` the reference's normaliser accepts."""
    from eth_b200.contract.config import uniform_config   # pure Python, no native library
    pp, tp, dp = layout
    cfg = uniform_config(model, pp=pp, tp=tp, dp=dp, gbs=gbs, mbs=micro_batch * dp)
    with open(path, "w") as f:
        json.dump(cfg, f, indent=1)


def reference_argv(config_path: str, log_dir: str, iters: int, dtype_flag: str, loss_scale, local_rank: int) -> list:
    """Arguments of scripts/train_gpt.sh:286-309 for block-wise sync with 32 MiB buckets, plus the
    `--local_rank` that `torch.distributed.launch` (the reference's launcher, :349) passes."""
    argv = [
        "pretrain_gpt.py", f"--local_rank={local_rank}", "--flexpipe-config", config_path, "--train-iters", str(iters), "--eval-iters", "0",
        "--lr-decay-iters", "320000", "--vocab-file", "vocabs/gpt2-vocab.json", "--merge-file",
        "vocabs/gpt2-merges.txt", "--data-impl", "mmap", "--split", "949,50,1", "--distributed-backend", "nccl",
        "--lr", "0.00015", "--lr-decay-style", "cosine", "--min-lr", "1.0e-5", "--weight-decay", "1e-2",
        "--clip-grad", "1.0", "--lr-warmup-fraction", ".01", "--log-interval", "1", "--DDP-impl", "local",
        "--grad-sync-mode", "block", "--grad-sync-bucket-size-mb", "32", "--grad-sync-metadata-transport",
        "auto", "--log-path", log_dir.rstrip("/") + "/", dtype_flag,
    ]
    if loss_scale:
        argv += ["--loss-scale", str(loss_scale)]
    return argv


class _StepTimer:
    """Wraps the reference's `train_step`; see the module docstring for what is timed."""

    def __init__(self, inner, warmup: int, steps: int):
        import torch
        self.torch, self.inner, self.warmup, self.steps = torch, inner, warmup, steps
        self.calls = 0
        self.pairs = []
        self.span = None
        self.on_window_start = self.on_window_end = None

    def _fence(self):
        torch = self.torch
        if torch.distributed.is_initialized():
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def __call__(self, *args, **kwargs):
        torch = self.torch
        i = self.calls
        if i == self.warmup:
            self._fence()
            if self.on_window_start:
                self.on_window_start()
            self.span = [torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)]
            self.span[0].record()
        if i == self.warmup + self.steps:
            # entry of the first call after the window: the last timed iteration's logging is done
            self.span[1].record()
            self._fence()
            if self.on_window_end:
                self.on_window_end()
        timed = self.warmup <= i < self.warmup + self.steps
        if timed:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
        out = self.inner(*args, **kwargs)
        if timed:
            e.record()
            self.pairs.append((s, e))
        self.calls += 1
        return out

    def results(self):
        torch = self.torch
        torch.cuda.synchronize()
        device_ms = sum(s.elapsed_time(e) for s, e in self.pairs)
        e2e_ms = self.span[0].elapsed_time(self.span[1])
        t = torch.tensor([device_ms, e2e_ms], device="cuda", dtype=torch.float64)
        if torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t[0].item()), float(t[1].item())


def _watch_for_peer_failure(flag_dir: str, rank: int):
    """A rank that fails leaves a file; the others stop waiting in their collectives and exit 0."""
    def loop():
        while True:
            time.sleep(1.0)
            try:
                names = [n for n in os.listdir(flag_dir) if n.startswith("fail_")]
            except OSError:
                return
            if names:
                if rank == 0:
                    try:
                        reason = open(os.path.join(flag_dir, sorted(names)[0])).read().strip()
                    except OSError:
                        reason = "a peer rank failed"
                    os.write(_REAL_STDOUT, (json.dumps({"impl": "reference", "unavailable": reason}) + "\n").encode())
                os._exit(0)
    threading.Thread(target=loop, daemon=True).start()


_REAL_STDOUT = 1


def run(opts, model, layouts, samples_per_gpu, micro_batch, vocab, clock_sampler_cls=None):
    global _REAL_STDOUT
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    profiling = os.environ.get("ETHB_REF_PROFILING", "0")
    os.environ["PROFILING"] = profiling

    def emit(obj):
        if rank == 0:
            os.write(_REAL_STDOUT, (json.dumps(obj) + "\n").encode())

    if not os.path.isfile(os.path.join(REF_RUNTIME, "pretrain_gpt.py")):
        emit({"impl": "reference", "unavailable": "baseline/_ref holds no copy of the reference tree"})
        return
    if world != opts.gpus:
        emit({"impl": "reference", "unavailable": f"--gpus {opts.gpus} but WORLD_SIZE={world}"})
        return

    # the reference prints freely; keep stdout for the one JSON line
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)

    work = os.path.join(tempfile.gettempdir(), f"ethb_ref_{os.environ['MASTER_PORT']}_{opts.gpus}")
    os.makedirs(work, exist_ok=True)
    if rank == 0:
        for n in os.listdir(work):
            if n.startswith("fail_"):
                os.unlink(os.path.join(work, n))
    _watch_for_peer_failure(work, rank)

    gbs = samples_per_gpu * opts.gpus
    layout = layouts[opts.gpus]
    config_path = os.path.join(work, f"gpt_bench_{opts.gpus}gpu.json")
    if local_rank == 0:
        write_config(config_path + ".tmp", model, layout, gbs, micro_batch)
        os.replace(config_path + ".tmp", config_path)
    else:
        deadline = time.time() + 60
        while not os.path.exists(config_path) and time.time() < deadline:
            time.sleep(0.1)

    shims = ["apex stub (torch AdamW fallback)", "sm_100 gencode appended to JIT flags", f"PROFILING={profiling}",
             "launcher script bypassed (CUDA 12.4 / Apex pin checks)"]
    restore_loader = None
    try:
        import torch
        iters = opts.warmup + opts.steps + 1
        dtype_flag = "--bf16" if getattr(opts, "bf16", False) else "--fp16"
        loss_scale = None if dtype_flag == "--bf16" else 4096
        sys.argv = reference_argv(config_path, os.path.join(work, "logs"), iters, dtype_flag, loss_scale, local_rank)
        os.makedirs(os.path.join(work, "logs", "csv"), exist_ok=True)   # the launcher creates it (scripts/train_gpt.sh)
        sys.path[:0] = [REF_RUNTIME, SHIMS]
        os.chdir(REF_RUNTIME)
        from baseline.reference_build import wrap_extension_loader
        build_log = []
        restore_loader = wrap_extension_loader(build_log)
        import importlib
        ref_main = importlib.import_module("pretrain_gpt")
        training = importlib.import_module("megatron.training")
        timer = _StepTimer(training.train_step, opts.warmup, opts.steps)
        sampler = clock_sampler_cls(local_rank) if (clock_sampler_cls and rank == 0) else None
        clocks = {}
        if sampler:
            timer.on_window_start = sampler.start
            timer.on_window_end = lambda: clocks.update(sampler.stop())
        training.train_step = timer
        ref_main.pretrain(ref_main.train_valid_test_datasets_provider, ref_main.model_provider,
                          ref_main.forward_step, args_defaults={"tokenizer_type": "GPT2BPETokenizer"})
        device_ms, e2e_ms = timer.results()
        pp, tp, dp = layout
        tokens = gbs * model["seq_length"] * opts.steps
        emit({
            "metric": "GPT training throughput (tokens/s, device-timed, max over ranks)",
            "value": tokens / (device_ms / 1e3), "unit": "tokens/s", "n_gpus": opts.gpus, "steps": opts.steps,
            "warmup": opts.warmup, "ms_per_step": device_ms / opts.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": dtype_flag[2:],
            "data": "synthetic token ids, random-init weights", "impl": "reference", "same_config": True,
            "config": {"model": "GPT-1.3B (24 layers, hidden 2048, 16 heads)", "global_batch": gbs,
                       "seq_len": model["seq_length"], "micro_batch": micro_batch, "pipeline_micro_batch": micro_batch * dp,
                       "parallelism": f"pp{pp}tp{tp}dp{dp}", "grad_sync": "block, 32 MiB buckets",
                       "l2": "inputs larger than L2 (each step streams several GB of weights and activations)"},
            "clocks": clocks or None,
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / opts.steps,
                    "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 12,
                    "note": "the reference builds its synthetic batch on the device; its per-iteration log reads "
                            "loss, loss scale and gradient norm back to the host"},
            "shims": shims + build_log,
        })
    except BaseException as exc:  # SystemExit from argparse included
        where = _first_reference_frame(exc)
        reason = f"{where}: {type(exc).__name__}: {str(exc).splitlines()[0] if str(exc) else ''}"[:400]
        traceback.print_exc(file=sys.stderr)
        try:
            with open(os.path.join(work, f"fail_{rank}"), "w") as f:
                f.write(reason)
        except OSError:
            pass
        emit({"impl": "reference", "unavailable": reason, "shims": shims})
        sys.stderr.flush()
        os._exit(0)
    finally:
        if restore_loader:
            restore_loader()
    sys.stderr.flush()
    # the reference leaves its process groups open; leave without running their destructors
    os._exit(0)
