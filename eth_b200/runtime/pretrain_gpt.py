"""GPT pretraining entry point: `python -m eth_b200.runtime.pretrain_gpt --flexpipe-config ...`
under `torch.distributed.run` (one process per GPU).

Flow (reference: eth/runtime/pretrain_gpt.py:164 -> megatron/training.py:94-190): parse flags and
the HPP config, initialise the process group, build this rank's stage / gradient sync / optimizer,
optionally load a checkpoint, check that all ranks agree on the training clock, train, report per
iteration, and write the per-rank CSV summary.
"""
from __future__ import annotations

import csv
import math
import os
import time

import torch
import torch.distributed as dist

from ..parallel.grad_sync.loss import validate_training_clock_states
from .arguments import parse_args
from .checkpointing import load_checkpoint, save_checkpoint
from ..data.provider import providers_from_args
from .engine import TrainEngine


def initialize_distributed(args):
    if args.device == "cpu" or not torch.cuda.is_available():
        device = torch.device("cpu")
        backend = "gloo"
    else:
        torch.cuda.set_device(args.local_rank % torch.cuda.device_count())
        device = torch.device("cuda", torch.cuda.current_device())
        backend = args.distributed_backend
    if args.world_size > 1 and not dist.is_initialized():
        kw = {"device_id": device} if backend == "nccl" else {}
        dist.init_process_group(backend, rank=args.rank, world_size=args.world_size, **kw)
        t = torch.ones(1, device=device)
        dist.all_reduce(t)   # communicator warm-up (reference: initialize.py:208-212)
    return device


def print_rank_0(*a):
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(*a, flush=True)


def training_log(engine, stats, elapsed_ms, total_ms, log_state):
    a = engine.args
    it = stats["iteration"]
    loss = engine.reduced_loss()
    log_state["skipped"] += 0 if stats["update_successful"] else 1
    if loss != loss:
        log_state["nan"] += 1
    line = (f" iteration {it:8d}/{a.train_iters:8d} | consumed samples: {engine.clock.successful_optimizer_steps * a.total_gbs:12d} | "
            f"elapsed time per iteration (ms): {elapsed_ms:.1f} | ")
    if it > 1:
        line += f"average (ms, excluding the first): {total_ms / (it - 1):.1f} | "
    tokens_per_s = a.total_gbs * a.seq_length / (elapsed_ms / 1e3)
    line += (f"tokens/s: {tokens_per_s:.1f} | learning rate: {stats['lr']:.3E} | global batch size: {a.total_gbs:5d} | "
             f"lm loss: {loss:.6E} | loss scale: {stats['loss_scale']:.1f} | ")
    if stats["grad_norm"] is not None:
        line += f"grad norm: {stats['grad_norm']:.3f} | "
    exposed = engine.exposed_grad_sync_ms()
    line += f"exposed grad sync (ms): {exposed:.2f} | "
    line += f"number of skipped iterations: {log_state['skipped']:3d} | number of nan iterations: {log_state['nan']:3d} |"
    if a.local_rank == 0:
        print(line, flush=True)
    if log_state.get("writer") is not None:
        w = log_state["writer"]
        samples = engine.clock.successful_optimizer_steps * a.total_gbs
        for key, val in (("learning-rate", stats["lr"]), ("lm loss", loss), ("loss-scale", stats["loss_scale"]),
                         ("grad-norm", stats["grad_norm"]), ("iteration-time-ms", elapsed_ms),
                         ("tokens-per-second", tokens_per_s), ("exposed-grad-sync-ms", exposed)):
            if val is not None:
                w.add_scalar(key, val, it)
                w.add_scalar(key + " vs samples", val, samples)
    return loss, tokens_per_s, exposed


def make_tensorboard_writer(args):
    """SummaryWriter on the last rank when `--tensorboard-dir` is given (reference:
    eth/runtime/megatron/global_vars.py:137-154); None elsewhere or when tensorboard is missing."""
    if not getattr(args, "tensorboard_dir", None) or args.rank != args.world_size - 1:
        return None
    try:
        from torch.utils.tensorboard import SummaryWriter
    except Exception:
        print("WARNING: tensorboard is not importable; no tensorboard logs will be written", flush=True)
        return None
    return SummaryWriter(log_dir=args.tensorboard_dir, max_queue=getattr(args, "tensorboard_queue_size", 1000))


def write_rank_csv(engine, rows):
    a, ps = engine.args, engine.pstate
    if not a.log_path:
        return
    os.makedirs(os.path.join(a.log_path, "csv"), exist_ok=True)
    name = f"{a.normalized_config['config_hash'][:12]}_stage{ps.stage_id}_rank{a.rank}.csv"
    mem = torch.cuda.max_memory_allocated() / 2 ** 20 if torch.cuda.is_available() else 0.0
    res = torch.cuda.max_memory_reserved() / 2 ** 20 if torch.cuda.is_available() else 0.0
    with open(os.path.join(a.log_path, "csv", name), "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["iteration", "ms_per_iteration", "tokens_per_s", "lm_loss", "grad_norm", "exposed_grad_sync_ms",
                    "max_allocated_mb", "max_reserved_mb"])
        for r in rows:
            w.writerow(list(r) + [f"{mem:.1f}", f"{res:.1f}"])


def evaluate(engine, eval_iters: int):
    """Mean masked LM loss and perplexity over `eval_iters` forward-only global batches
    (reference: eth/runtime/megatron/training.py:1399-1475). Evaluation batches are drawn after the
    training cursor without advancing it."""
    total, weight = 0.0, 0.0
    cursor = engine.clock.global_data_cursor
    # a validation dataset is read from its own position, which moves on from one evaluation to the next
    own_cursor = engine.eval_data_provider is not None and engine.eval_data_provider is not engine.data_provider
    if own_cursor:
        engine.clock.global_data_cursor = engine.eval_cursor
    try:
        for _ in range(eval_iters):
            engine.eval_step()
            s, w = engine.loss_acc.tolist()
            total, weight = total + s, weight + w
            engine.clock.global_data_cursor += engine.clock.total_gbs
        if own_cursor:
            engine.eval_cursor = engine.clock.global_data_cursor
    finally:
        engine.clock.global_data_cursor = cursor
    loss = total / weight if weight > 0 else float("nan")
    return {"lm loss": loss, "lm loss ppl": math.exp(min(20.0, loss)) if loss == loss else float("nan")}


def pretrain(argv=None):
    args = parse_args(argv)
    device = initialize_distributed(args)
    t_start = time.time()
    engine = TrainEngine(args, device=device)
    engine.data_provider, engine.eval_data_provider = providers_from_args(args, engine.pstate, args.eod_token)
    if args.data_path:
        print_rank_0(f"> training on {args.data_path} (split {args.split}); validation set: "
                     f"{'yes' if engine.eval_data_provider is not None else 'none'}")
    if args.load:
        load_checkpoint(engine, args.load)
        if args.eval_interval:   # validation data already read by the evaluations before the checkpoint
            engine.eval_cursor = (engine.iteration // args.eval_interval) * args.eval_iters * args.total_gbs
    # all ranks must agree on the clock before the first step (reference: training.py:896-898)
    states = [None] * args.world_size
    engine.coll.all_gather_object(states, (engine.clock.global_data_cursor, engine.clock.successful_optimizer_steps))
    validate_training_clock_states(states)
    print_rank_0(f"> model and optimizer ready in {time.time() - t_start:.1f} s "
                 f"({sum(p.numel() for _, p in engine.stage.named_parameters()) / 1e6:.1f} M parameters on rank 0)")
    log_state = {"skipped": 0, "nan": 0, "writer": make_tensorboard_writer(args)}
    rows, total_ms = [], 0.0
    use_cuda = device.type == "cuda"
    while engine.iteration < args.train_iters:
        if use_cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
        t0 = time.perf_counter()
        stats = engine.train_step()
        if use_cuda:
            e.record()
            e.synchronize()
            ms = s.elapsed_time(e)
        else:
            ms = (time.perf_counter() - t0) * 1e3
        if stats["iteration"] > 1:
            total_ms += ms
        if stats["iteration"] % args.log_interval == 0:
            loss, tps, exposed = training_log(engine, stats, ms, total_ms, log_state)
            rows.append((stats["iteration"], f"{ms:.2f}", f"{tps:.1f}", f"{loss:.6f}", stats["grad_norm"], f"{exposed:.3f}"))
        if args.eval_iters and args.eval_interval and engine.iteration % args.eval_interval == 0:
            res = evaluate(engine, args.eval_iters)
            print_rank_0(f" validation loss at iteration {engine.iteration} | lm loss value: {res['lm loss']:.6E} | "
                         f"lm loss PPL: {res['lm loss ppl']:.6E}")
        if args.save and args.save_interval and engine.iteration % args.save_interval == 0:
            save_checkpoint(engine, engine.iteration, args.save)
        if args.exit_interval and engine.iteration % args.exit_interval == 0:
            if args.save:
                save_checkpoint(engine, engine.iteration, args.save)
            print_rank_0(f"exiting program at iteration {engine.iteration}")
            break
        if args.exit_duration_in_mins and (time.time() - t_start) / 60.0 > args.exit_duration_in_mins:
            if args.save:
                save_checkpoint(engine, engine.iteration, args.save)
            print_rank_0(f"exiting program after {(time.time() - t_start) / 60.0:.1f} minutes")
            break
    if args.save and (not args.save_interval or engine.iteration % args.save_interval):
        save_checkpoint(engine, engine.iteration, args.save)
    write_rank_csv(engine, rows)
    if log_state["writer"] is not None:
        log_state["writer"].close()
    if use_cuda:
        from ..ops import native
        native.check_status()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return engine


if __name__ == "__main__":
    pretrain()
