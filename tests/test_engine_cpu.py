"""The explicit stage program against a plain autograd GPT, and one optimizer step against AdamW."""
import math

import pytest
import torch

from eth_b200.contract.config import make_config, make_pipe, manifest_size
from eth_b200.runtime.arguments import parse_args
from eth_b200.runtime.engine import TrainEngine
from tests.helpers.oracle_gpt import oracle_loss


def _args(cfg, extra=()):
    argv = ["--hidden-dropout", "0.0", "--device", "cpu", "--vocab-size", "200",
            "--make-vocab-size-divisible-by", "8"] + list(extra)
    return parse_args(argv, config=cfg, rank=0, world_size=1)


def _tiny(recompute=None, layers=2, gbs=4, mbs=2):
    n = manifest_size(layers)
    pipe = make_pipe([n], [1], [1], gbs=gbs, mbs=mbs, recompute=recompute)
    return make_config([pipe], num_layers=layers, hidden_size=32, num_attention_heads=4, seq_length=16)


@pytest.mark.parametrize("recompute", [False, True])
def test_gradients_match_autograd(recompute):
    torch.manual_seed(0)
    layers = 2
    n = manifest_size(layers)
    rec = [[1 if 1 <= i <= 14 else 0 for i in range(n)]] if recompute else None
    args = _args(_tiny(rec, layers))
    eng = TrainEngine(args, device="cpu")
    cfg = eng.model_cfg
    params = {lid: p.detach().clone().float().requires_grad_(True) for lid, p in eng.stage.named_parameters()}
    # oracle over the same micro-batches
    total = 0.0
    for i in range(eng.pstate.num_microbatches):
        tokens, labels, mask = eng.get_batch(i)
        l, _ = oracle_loss(params, tokens, labels, mask, cfg, args.nominal_global_loss_scale)
        total = total + l
    total.backward()
    eng.optimizer.zero_grad()
    eng.loss_acc.zero_()
    from eth_b200.runtime import schedules
    schedules.forward_backward_no_pipelining(eng, eng.pstate.num_microbatches)
    for lid, p in eng.stage.named_parameters():
        ref = params[lid].grad
        err = (p.main_grad - ref).norm() / (ref.norm() + 1e-12)
        assert err < 1e-4, (lid, float(err))
    assert abs(float(eng.loss_acc[0]) / args.nominal_global_loss_scale - float(total)) < 1e-4


def test_train_step_matches_adamw():
    args = _args(_tiny(), ["--clip-grad", "1.0", "--lr", "1e-3", "--lr-warmup-fraction", "0.0",
                           "--lr-decay-style", "constant"])
    eng = TrainEngine(args, device="cpu")
    cfg = eng.model_cfg
    params = {lid: p.detach().clone().float().requires_grad_(True) for lid, p in eng.stage.named_parameters()}
    decay = [v for k, v in params.items() if k.endswith("weight") and "layernorm" not in k]
    nodecay = [v for k, v in params.items() if not (k.endswith("weight") and "layernorm" not in k)]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.01}, {"params": nodecay, "weight_decay": 0.0}],
                            lr=1e-3, betas=(0.9, 0.999), eps=1e-8)
    for step in range(2):
        opt.zero_grad()
        total, wsum = 0.0, 0.0
        eng.clock.global_data_cursor  # data cursor is advanced by the engine itself
        for i in range(eng.pstate.num_microbatches):
            tokens, labels, mask = eng.get_batch(i)
            l, _ = oracle_loss(params, tokens, labels, mask, cfg, 1.0)
            total = total + l
            wsum += float(mask.sum())
        (total / wsum).backward()
        gn = torch.nn.utils.clip_grad_norm_(list(params.values()), 1.0)
        opt.step()
        stats = eng.train_step()
        assert stats["update_successful"]
        assert abs(stats["grad_norm"] - float(gn)) / float(gn) < 1e-3
        assert abs(eng.reduced_loss() - float(total) / wsum) < 1e-4
    for lid, p in eng.stage.named_parameters():
        err = (p - params[lid]).norm() / (params[lid].norm() + 1e-12)
        assert err < 1e-4, (lid, float(err))


@pytest.mark.parametrize("recompute", [False, True])
def test_dropout_add_fused_into_the_gemm_trains_like_the_separate_op(recompute):
    """With hidden dropout on, the bias-dropout-add that runs in the epilogue of the row-parallel
    GEMM draws the mask of the stand-alone op: a stage built with fusions and one built without
    produce the same loss and the same gradients, also when the fused pair is recomputed."""
    from eth_b200.runtime import schedules
    layers = 2
    n = manifest_size(layers)
    rec = [[1 if 1 <= i <= 14 else 0 for i in range(n)]] if recompute else None
    results = []
    for fuse in (True, False):
        args = _args(_tiny(rec, layers), ["--hidden-dropout", "0.2"])
        eng = TrainEngine(args, device="cpu")
        fused_ops = [op for op in eng.stage.ops if getattr(op, "fused_dropout_add", None) is not None]
        assert len(fused_ops) == 2 * layers
        if not fuse:
            for op in fused_ops:
                op.fused_dropout_add = None
        eng.optimizer.zero_grad()
        eng.loss_acc.zero_()
        schedules.forward_backward_no_pipelining(eng, eng.pstate.num_microbatches)
        results.append((float(eng.loss_acc[0]), {lid: p.main_grad.clone() for lid, p in eng.stage.named_parameters()}))
    (loss_a, grads_a), (loss_b, grads_b) = results
    assert abs(loss_a - loss_b) < 1e-5 * abs(loss_b)
    for lid in grads_a:
        err = (grads_a[lid] - grads_b[lid]).norm() / (grads_b[lid].norm() + 1e-12)
        assert err < 1e-5, (lid, float(err))
