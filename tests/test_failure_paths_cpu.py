"""Failure detection, exercised on the host only: every failure here is made by a CPU rank (one that
leaves, one that lies about its metadata) or by a damaged file; no device is involved."""
import datetime
import os
import tempfile
from dataclasses import replace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from eth_b200.contract.config import make_config, make_pipe, manifest_size
from tests.helpers.multiproc import _free_port, run_ranks

LAYERS = 2


def _dp2_engine(rank, world):
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    cfg = make_config([make_pipe([manifest_size(LAYERS)], [1], [world], gbs=4, mbs=2)], num_layers=LAYERS,
                      hidden_size=32, num_attention_heads=4, seq_length=16)
    args = parse_args(["--hidden-dropout", "0.0", "--device", "cpu", "--vocab-size", "64", "--lr", "1e-2",
                       "--make-vocab-size-divisible-by", "8", "--distributed-backend", "gloo"],
                      config=cfg, rank=rank, world_size=world)
    return TrainEngine(args, device="cpu")


# ------------------------------------------------------------------ a rank leaves between steps
def _leaver_worker(rank, world, port, outdir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    report = {"steps": 0, "error": None}
    try:
        eng = _dp2_engine(rank, world)
        eng.train_step()
        report["steps"] = 1
        if rank == 1:
            # leaves between steps: nothing of its own is in flight
            torch.save(report, os.path.join(outdir, f"rank{rank}.pt"))
            dist.destroy_process_group()
            return
        try:
            eng.train_step()           # the next collective has no partner any more
            report["steps"] = 2
        except Exception as err:       # noqa: BLE001 - the point of the test is that *an* error surfaces
            report["error"] = f"{type(err).__name__}: {str(err)[:200]}"
    finally:
        torch.save(report, os.path.join(outdir, f"rank{rank}.pt"))


def test_survivor_gets_an_error_when_its_partner_leaves_between_steps():
    port = _free_port()
    with tempfile.TemporaryDirectory() as outdir:
        ctx = mp.get_context("spawn")
        procs = [ctx.Process(target=_leaver_worker, args=(r, 2, port, outdir)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
        alive = [p for p in procs if p.is_alive()]
        for p in alive:
            p.terminate()
        assert not alive, "the surviving rank hung instead of failing"
        left = torch.load(os.path.join(outdir, "rank1.pt"), weights_only=False)
        stayed = torch.load(os.path.join(outdir, "rank0.pt"), weights_only=False)
        assert left["steps"] == 1 and left["error"] is None
        assert stayed["steps"] == 1 and stayed["error"], stayed


# ------------------------------------------------------------------ a rank publishes a wrong descriptor
def _lying_rank(rank, world):
    from eth_b200.parallel.grad_sync import manager as M
    real_gather = None

    eng_error = None
    original = M.plan_canonical_fragments

    def tampered(descriptors, expected_pipeline_ids):
        # what rank 1 told the world about one weight is wrong (as if its metadata were corrupted in
        # transit): every rank plans from the same gathered list, so every rank must refuse it
        descriptors = [replace(d, full_shape=(d.full_shape[0] + 8,) + tuple(d.full_shape[1:]))
                       if d.global_rank == 1 and d.logical_param_id.endswith("mlp.dense_h_to_4h.weight") else d
                       for d in descriptors]
        return original(descriptors, expected_pipeline_ids)

    M.plan_canonical_fragments = tampered
    try:
        _dp2_engine(rank, world)
    except ValueError as err:
        eng_error = str(err)
    finally:
        M.plan_canonical_fragments = original
    del real_gather
    return eng_error


def test_corrupted_descriptor_is_rejected_on_every_rank():
    errors = run_ranks(2, _lying_rank)
    assert all(e and "shape mismatch" in e for e in errors), errors


# ------------------------------------------------------------------ a damaged checkpoint
def test_truncated_checkpoint_is_reported_not_loaded(tmp_path):
    from eth_b200.runtime.checkpointing import load_checkpoint, save_checkpoint
    eng = _dp2_engine(0, 1)
    eng.train_step()
    path = save_checkpoint(eng, eng.iteration, str(tmp_path))
    size = os.path.getsize(path)
    with open(path, "r+b") as f:
        f.truncate(size // 2)
    before = eng.stage.param_buf.clone()
    fresh = _dp2_engine(0, 1)
    with pytest.raises(RuntimeError, match="could not load checkpoint"):
        load_checkpoint(fresh, str(tmp_path))
    assert fresh.iteration == 0 and fresh.clock.global_data_cursor == 0     # nothing half-applied
    assert torch.equal(eng.stage.param_buf, before)


def test_device_fault_mark_travels_with_the_overflow_flag():
    """The optimizer's control block carries 'some rank saw a device time-out' next to the overflow
    flag; a marked step is skipped and reported, and the loss scaler is not punished for it."""
    from eth_b200.optim.optimizer import DEVICE_FAULT_MARK
    eng = _dp2_engine(0, 1)
    eng.train_step()
    opt = eng.optimizer
    real = opt.compute_norm_and_inf

    def with_fault():
        real()
        opt.ctrl[1] += DEVICE_FAULT_MARK      # what a rank with a non-zero status word adds

    opt.compute_norm_and_inf = with_fault
    before = eng.stage.param_buf.clone()
    with pytest.raises(RuntimeError, match="bounded device wait"):
        eng.train_step()
    assert torch.equal(eng.stage.param_buf, before)
