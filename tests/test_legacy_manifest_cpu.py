"""The 13-op layer manifest (unfused attention: score, softmax, dropout, context) as a runnable stage
program: same loss and gradients as the 10-op manifest with its fused attention op, and as the
autograd oracle."""
import pytest
import torch

from eth_b200.contract.config import (LEGACY_LAYER_OPS, make_config, make_pipe, manifest_size,
                                      normalize_flexpipe_config)
from eth_b200.runtime import schedules
from eth_b200.runtime.arguments import parse_args
from eth_b200.runtime.engine import TrainEngine

LAYERS = 2


def _engine(impl, extra=()):
    n = manifest_size(LAYERS, impl)
    cfg = make_config([make_pipe([n], [1], [1], gbs=4, mbs=2)], num_layers=LAYERS, hidden_size=32,
                      num_attention_heads=4, seq_length=16)
    cfg["model_impl"] = impl
    args = parse_args(["--hidden-dropout", "0.0", "--device", "cpu", "--vocab-size", "200",
                       "--make-vocab-size-divisible-by", "8"] + list(extra), config=cfg, rank=0, world_size=1)
    return TrainEngine(args, device="cpu")


def _grads(eng):
    eng.optimizer.zero_grad()
    eng.loss_acc.zero_()
    schedules.forward_backward_no_pipelining(eng, eng.pstate.num_microbatches)
    return {lid: p.main_grad.clone() for lid, p in eng.stage.named_parameters()}, float(eng.loss_acc[0])


def test_manifest_has_thirteen_ops_per_layer_and_its_own_hash():
    assert manifest_size(LAYERS, "gpt-legacy13") == 3 + 13 * LAYERS
    fused, legacy = _engine("gpt"), _engine("gpt-legacy13")
    names = [op.name for op in legacy.stage.ops]
    assert names[1:14] == list(LEGACY_LAYER_OPS) and len(names) == 3 + 13 * LAYERS
    assert legacy.args.normalized_config["manifest"]["hash"] != fused.args.normalized_config["manifest"]["hash"]
    assert legacy.args.normalized_config["model_impl"] == "gpt-legacy13"
    # the op count alone identifies the manifest
    n = manifest_size(LAYERS, "gpt-legacy13")
    cfg = make_config([make_pipe([n], [1], [1], gbs=4, mbs=2)], num_layers=LAYERS, hidden_size=32,
                      num_attention_heads=4, seq_length=16)
    cfg.pop("model_impl", None)
    with pytest.warns(UserWarning, match="inferred"):
        assert normalize_flexpipe_config(cfg)["model_impl"] == "gpt-legacy13"


def test_unfused_attention_ops_match_the_fused_op():
    torch.manual_seed(0)
    fused, legacy = _engine("gpt"), _engine("gpt-legacy13")
    for (la, pa), (lb, pb) in zip(fused.stage.named_parameters(), legacy.stage.named_parameters()):
        assert la == lb and torch.equal(pa, pb)          # same logical parameters, same init
    g_fused, loss_fused = _grads(fused)
    g_legacy, loss_legacy = _grads(legacy)
    assert abs(loss_fused - loss_legacy) < 1e-4 * abs(loss_fused)
    for lid, ref in g_fused.items():
        err = (g_legacy[lid] - ref).norm() / (ref.norm() + 1e-12)
        assert err < 1e-4, (lid, float(err))


def test_attention_dropout_is_an_op_of_the_legacy_manifest_only():
    with pytest.raises(ValueError, match="attention-dropout"):
        _engine("gpt", ["--attention-dropout", "0.1"])
    eng = _engine("gpt-legacy13", ["--attention-dropout", "0.1"])
    g1, l1 = _grads(eng)
    g2, l2 = _grads(eng)                       # same step, same micro-batches: the same mask is drawn
    assert l1 == l2 and all(torch.equal(g1[k], g2[k]) for k in g1)
    plain, l0 = _grads(_engine("gpt-legacy13"))
    assert abs(l0 - l1) > 1e-6                 # and the mask does change the result


def test_stage_boundary_inside_the_unfused_block_is_refused():
    n = manifest_size(LAYERS, "gpt-legacy13")
    cfg = make_config([make_pipe([4, n - 4], [1, 1], [1, 1], gbs=4, mbs=2)], num_layers=LAYERS, hidden_size=32,
                      num_attention_heads=4, seq_length=16)
    cfg["model_impl"] = "gpt-legacy13"
    args = parse_args(["--device", "cpu", "--vocab-size", "200", "--make-vocab-size-divisible-by", "8"], config=cfg,
                      rank=0, world_size=2)
    with pytest.raises(ValueError, match="unfused attention block"):
        TrainEngine(args, device="cpu")
