"""Checkpoint layout and resume equivalence on CPU."""
import os

import torch

from eth_b200.contract.config import make_config, make_pipe, manifest_size
from eth_b200.runtime.arguments import parse_args
from eth_b200.runtime.checkpointing import checkpoint_name, load_checkpoint, read_tracker, save_checkpoint
from eth_b200.runtime.engine import TrainEngine


def _engine():
    layers = 2
    cfg = make_config([make_pipe([manifest_size(layers)], [1], [1], gbs=4, mbs=2)], num_layers=layers,
                      hidden_size=32, num_attention_heads=4, seq_length=16)
    args = parse_args(["--hidden-dropout", "0.0", "--device", "cpu", "--vocab-size", "64", "--lr", "1e-2",
                       "--make-vocab-size-divisible-by", "8", "--lr-warmup-fraction", "0.0"], config=cfg, rank=0, world_size=1)
    return TrainEngine(args, device="cpu")


def test_layout_names():
    assert checkpoint_name("/x", 12, 3, 0, 1).endswith("iter_0000012/mp_rank_03/model_optim_rng.pt")
    assert checkpoint_name("/x", 12, 3, 5, 8).endswith("iter_0000012/mp_rank_03_005/model_optim_rng.pt")
    assert checkpoint_name("/x", 0, 0, 0, 1, release=True).endswith("release/mp_rank_00/model_optim_rng.pt")


def test_resume_is_bit_identical(tmp_path):
    a = _engine()
    a.train_step(); a.train_step()
    path = save_checkpoint(a, a.iteration, str(tmp_path))
    assert os.path.isfile(path) and read_tracker(str(tmp_path)) == (2, False)
    state = torch.load(path, weights_only=False)
    assert state["checkpoint_version"] == 3.0 and state["iteration"] == 2
    assert {"args", "model", "optimizer", "lr_scheduler", "torch_rng_state"} <= set(state)
    a.train_step()
    b = _engine()
    assert load_checkpoint(b, str(tmp_path)) == 2
    assert b.clock.global_data_cursor == 8 and b.clock.successful_optimizer_steps == 2
    b.train_step()
    for (la, pa), (lb, pb) in zip(a.stage.named_parameters(), b.stage.named_parameters()):
        assert la == lb and torch.equal(pa, pb), la


def _fp16_dp2_resume(rank, world, root):
    """Two data-parallel fp16 ranks: train, save, then resume in fresh engines that were built with
    a different initial loss scale. Only rank 0 reads the file; the scaler state and the schedule
    position must reach rank 1 as well."""
    from eth_b200.contract.config import make_config, make_pipe, manifest_size
    layers = 2
    cfg = make_config([make_pipe([manifest_size(layers)], [1], [2], gbs=4, mbs=2)], num_layers=layers,
                      hidden_size=32, num_attention_heads=4, seq_length=16)
    common = ["--fp16", "--hidden-dropout", "0.0", "--device", "cpu", "--vocab-size", "64", "--lr", "1e-2",
              "--make-vocab-size-divisible-by", "8", "--lr-warmup-fraction", "0.5", "--lr-decay-iters", "8",
              "--distributed-backend", "gloo", "--loss-scale-window", "2"]
    a = TrainEngine(parse_args(common + ["--initial-loss-scale", "1024"], config=cfg, rank=rank, world_size=world),
                    device="cpu")
    for _ in range(3):
        a.train_step()
    saved_scale, saved_lr = a.scaler.value(), a.optimizer.lr
    save_checkpoint(a, a.iteration, root)
    b = TrainEngine(parse_args(common + ["--initial-loss-scale", "65536"], config=cfg, rank=rank, world_size=world),
                    device="cpu")
    assert load_checkpoint(b, root) == 3
    resumed = (b.scaler.value(), b.scaler.state_dict(), b.optimizer.lr, b.lr_scheduler.num_steps)
    a.train_step()
    b.train_step()
    same = all(torch.equal(pa, pb) for (_, pa), (_, pb) in zip(a.stage.named_parameters(), b.stage.named_parameters()))
    flat = torch.cat([p.detach().float().reshape(-1) for _, p in b.stage.named_parameters()])
    return {"saved": (saved_scale, saved_lr), "resumed": resumed, "same_as_uninterrupted": same, "params": flat}


def test_fp16_dp2_resume_restores_scaler_on_every_rank(tmp_path):
    from tests.helpers.multiproc import run_ranks
    r0, r1 = run_ranks(2, _fp16_dp2_resume, str(tmp_path))
    assert r0["saved"][0] != 65536.0            # the scale moved away from both initial values
    for r in (r0, r1):
        assert r["resumed"][0] == r0["saved"][0] and r["resumed"][2] == r0["saved"][1]
        assert r["same_as_uninterrupted"]
    assert r0["resumed"] == r1["resumed"]
    assert torch.equal(r0["params"], r1["params"])
