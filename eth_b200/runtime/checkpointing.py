"""Checkpoint save / load.

Layout (reference: eth/runtime/megatron/checkpointing.py:84-107):
    <save>/latest_checkpointed_iteration.txt
    <save>/iter_<7 digits>/mp_rank_<tp:02d>[_<pp:03d>]/model_optim_rng.pt
written by the DP-rank-0 ranks only (:120). Contents (:122-153): args, checkpoint_version 3.0,
iteration, model, optimizer, lr_scheduler, python / numpy / torch / cuda RNG states, and the
training clock (`global_data_cursor`, `successful_optimizer_steps`, :331-334).

The reference's file name carries no pipeline index, so several pipelines overwrite each other.
Here only pipeline 0 writes and reads: after a load, parameters and optimizer moments are
re-broadcast fragment by fragment from each fragment's smallest rank (which lies in pipeline 0,
DP rank 0), so every other holder -- other DP replicas, other pipelines with other TP layouts --
receives exactly the loaded state.
"""
from __future__ import annotations

import os
import random
from types import SimpleNamespace

import numpy as np
import torch

CHECKPOINT_VERSION = 3.0


def tracker_filename(root: str) -> str:
    return os.path.join(root, "latest_checkpointed_iteration.txt")


def checkpoint_name(root: str, iteration, tp_rank: int, pp_rank: int, pp_size: int, release: bool = False) -> str:
    directory = "release" if release else "iter_{:07d}".format(iteration)
    if pp_size == 1:
        return os.path.join(root, directory, "mp_rank_{:02d}".format(tp_rank), "model_optim_rng.pt")
    return os.path.join(root, directory, "mp_rank_{:02d}_{:03d}".format(tp_rank, pp_rank), "model_optim_rng.pt")


def read_tracker(root: str):
    path = tracker_filename(root)
    if not os.path.isfile(path):
        return None, False
    text = open(path).read().strip()
    if text == "release":
        return 0, True
    try:
        return int(text), False
    except ValueError as exc:
        raise ValueError(f"invalid metadata file {path}: {text!r}") from exc


def _serialisable_args(args):
    keep = {}
    for k, v in vars(args).items():
        if isinstance(v, (int, float, str, bool, type(None), list, tuple, dict)):
            keep[k] = v
    return SimpleNamespace(**keep)


def is_writer(pstate) -> bool:
    return pstate.pipeline_id == 0 and pstate.dp_rank == 0


def save_checkpoint(engine, iteration: int, root: str) -> str:
    ps, args = engine.pstate, engine.args
    path = checkpoint_name(root, iteration, ps.tp_rank, ps.stage_id, ps.num_stages)
    if engine.device.type == "cuda":
        # A bounded device wait that ran out leaves stale gradients or partial GEMM outputs behind;
        # nothing computed from them may reach a checkpoint. All ranks agree before anyone writes.
        from ..ops import native
        fault = (native.status(engine.device) != 0).to(torch.float32)
        engine.coll.all_reduce_max(fault)
        if float(fault.item()) != 0.0:
            native.check_status(engine.device)   # raises with this rank's reason if it is the one
            raise RuntimeError("checkpoint not written: another rank reported a device kernel time-out")
    if is_writer(ps):
        args.global_data_cursor = engine.clock.global_data_cursor
        args.successful_optimizer_steps = engine.clock.successful_optimizer_steps
        args.consumed_train_samples = engine.clock.successful_optimizer_steps * args.total_gbs
        state = {
            "args": _serialisable_args(args), "checkpoint_version": CHECKPOINT_VERSION, "iteration": iteration,
            "model": {lid: p.detach().cpu() for lid, p in engine.stage.named_parameters()},
            "lr_scheduler": engine.lr_scheduler.state_dict(),
        }
        if not getattr(args, "no_save_optim", False):
            osd = engine.optimizer.state_dict()
            state["optimizer"] = {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in osd.items()}
        if not getattr(args, "no_save_rng", False):
            state["random_rng_state"] = random.getstate()
            state["np_rng_state"] = np.random.get_state()
            state["torch_rng_state"] = torch.get_rng_state()
            state["cuda_rng_state"] = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
            state["rng_tracker_states"] = {"dropout_seed": args.seed}
        os.makedirs(os.path.dirname(path), exist_ok=True)
        tmp = path + ".tmp"
        torch.save(state, tmp)
        os.replace(tmp, path)
    engine.coll.barrier()
    if engine.args.rank == 0:
        with open(tracker_filename(root), "w") as f:
            f.write(str(iteration))
    engine.coll.barrier()
    return path


def load_checkpoint(engine, root: str) -> int:
    """Restores model, optimizer, scheduler and clocks; returns the iteration (0 if none found)."""
    ps, args = engine.pstate, engine.args
    iteration, release = read_tracker(root)
    if iteration is None:
        return 0
    if is_writer(ps):
        path = checkpoint_name(root, iteration, ps.tp_rank, ps.stage_id, ps.num_stages, release)
        try:
            state = torch.load(path, map_location="cpu", weights_only=False)
        except Exception as exc:
            raise RuntimeError(f"could not load checkpoint {path}: {exc}") from exc
        params = dict(engine.stage.named_parameters())
        missing = set(params) - set(state["model"])
        if missing:
            raise KeyError(f"checkpoint {path} lacks parameters: {sorted(missing)[:4]} ...")
        for lid, p in params.items():
            src = state["model"][lid]
            if tuple(src.shape) != tuple(p.shape):
                raise ValueError(f"checkpoint shape mismatch for {lid}: {tuple(src.shape)} vs {tuple(p.shape)}")
            p.copy_(src.to(p.dtype))
        finetune = getattr(args, "finetune", False)
        if not finetune and not getattr(args, "no_load_optim", False) and "optimizer" in state:
            engine.optimizer.load_state_dict(state["optimizer"])
            engine.lr_scheduler.load_state_dict(state["lr_scheduler"])
        else:
            engine.optimizer.reload_model_params()
        if not finetune and not getattr(args, "no_load_rng", False) and "torch_rng_state" in state:
            random.setstate(state["random_rng_state"])
            np.random.set_state(state["np_rng_state"])
            torch.set_rng_state(state["torch_rng_state"])
        ck = state.get("args", SimpleNamespace())
        scaler = engine.optimizer.grad_scaler
        clock = [getattr(ck, "global_data_cursor", getattr(ck, "consumed_train_samples", 0)),
                 getattr(ck, "successful_optimizer_steps", iteration), 0 if finetune else state.get("iteration", iteration),
                 engine.optimizer.step_count,
                 scaler.state_dict() if scaler is not None else None,
                 engine.lr_scheduler.state_dict()]
    else:
        clock = None
    # Every rank learns the clocks, the loss-scaler state and the schedule position from rank 0 (a
    # writer); tensors follow through the fragment broadcasts below. Without the scaler state a
    # resumed fp16 job would scale its loss by the saved value on the writers and by the initial
    # value everywhere else, and the bucket sums would mix the two.
    box = [clock]
    if engine.coll.enabled:
        import torch.distributed as dist
        dist.broadcast_object_list(box, src=0)
    cursor, steps, it, opt_steps, scaler_state, lr_state = box[0]
    engine.clock.global_data_cursor, engine.clock.successful_optimizer_steps = cursor, steps
    engine.optimizer.step_count = opt_steps
    engine.iteration = it
    if not is_writer(ps):
        if engine.optimizer.grad_scaler is not None and scaler_state is not None:
            engine.optimizer.grad_scaler.load_state_dict(scaler_state)
        engine.lr_scheduler.load_state_dict(lr_state)
    bc = lambda t, src, handle: engine.coll.broadcast(t, src, group=handle)  # noqa: E731
    engine.grad_sync.synchronize_parameters(bc)
    engine.grad_sync.synchronize_optimizer_state(
        engine.optimizer, bc, lambda out, obj, handle: engine.coll.all_gather_object(out, obj, group=handle))
    engine.coll.barrier()
    return it
