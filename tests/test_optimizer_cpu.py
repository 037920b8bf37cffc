"""Flat optimizers against torch.optim on a fake stage (CPU)."""
import types

import torch

from eth_b200.optim.optimizer import FlatMixedPrecisionAdam, coalesce_ranges, get_optimizer
from eth_b200.optim.sgd import FlatSGD


def _stage(n=1000, decay=600, dtype=torch.float32):
    torch.manual_seed(0)
    st = types.SimpleNamespace()
    st.param_buf = torch.randn(n, dtype=dtype)
    st.grad_buf = torch.zeros(n, dtype=torch.float32)
    st.total_numel, st.decay_numel = n, decay
    st.zero_grad_buffer = lambda: st.grad_buf.zero_()
    return st


def _run(opt, st, ref_params, ref_opt, steps=4, clip=1.0):
    for i in range(steps):
        g = torch.randn(st.total_numel) * (3.0 if i == 1 else 0.1)
        st.grad_buf.copy_(g)
        ok, norm, _ = opt.step(sync=True)
        assert ok
        for p in ref_params:
            p.grad = None
        ref_params[0].grad = g[:st.decay_numel].clone()
        ref_params[1].grad = g[st.decay_numel:].clone()
        ref_norm = torch.nn.utils.clip_grad_norm_(ref_params, clip)
        assert abs(norm - float(ref_norm)) < 1e-4 * max(1.0, float(ref_norm))
        ref_opt.step()
        torch.testing.assert_close(st.param_buf[:st.decay_numel], ref_params[0].data, rtol=2e-5, atol=2e-6)
        torch.testing.assert_close(st.param_buf[st.decay_numel:], ref_params[1].data, rtol=2e-5, atol=2e-6)


def test_flat_adam_matches_torch_adamw():
    st = _stage()
    a = torch.nn.Parameter(st.param_buf[:600].clone())
    b = torch.nn.Parameter(st.param_buf[600:].clone())
    ref = torch.optim.AdamW([{"params": [a], "weight_decay": 0.01}, {"params": [b], "weight_decay": 0.0}],
                            lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    opt = FlatMixedPrecisionAdam(st, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01, clip_grad=1.0)
    _run(opt, st, [a, b], ref)


def test_flat_sgd_matches_torch_sgd():
    st = _stage()
    a = torch.nn.Parameter(st.param_buf[:600].clone())
    b = torch.nn.Parameter(st.param_buf[600:].clone())
    ref = torch.optim.SGD([{"params": [a], "weight_decay": 0.01}, {"params": [b], "weight_decay": 0.0}],
                          lr=1e-2, momentum=0.9)
    opt = FlatSGD(st, lr=1e-2, momentum=0.9, weight_decay=0.01, clip_grad=1.0)
    _run(opt, st, [a, b], ref)
    sd = opt.state_dict()
    assert "momentum_buffer" in sd and "exp_avg" not in sd
    opt.load_state_dict(sd)


def test_sgd_skips_on_overflow_and_factory():
    st = _stage()
    before = st.param_buf.clone()
    args = types.SimpleNamespace(optimizer="sgd", lr=0.1, sgd_momentum=0.5, weight_decay=0.0, clip_grad=0.0)
    opt = get_optimizer(st, args)
    assert isinstance(opt, FlatSGD)
    st.grad_buf.fill_(1.0)
    st.grad_buf[3] = float("inf")
    ok, _, _ = opt.step(sync=True)
    assert not ok and torch.equal(st.param_buf, before)
    # async mode: the kernels (here: the masked flat update) skip on their own
    ok, _, _ = opt.step(sync=False)
    assert torch.equal(st.param_buf, before)
    assert coalesce_ranges([(0, 10), (10, 5), (200, 4)]) == [(0, 15), (200, 4)]


def test_learning_rate_schedule_and_checkpoint_policy():
    import math
    import pytest
    from eth_b200.optim.lr import AnnealingLR, Schedule

    class Opt:
        lr = None

        def set_lr(self, v):
            self.lr = v

    s = Schedule(1e-2, 1e-3, warmup_steps=10, decay_steps=110, style="cosine")
    assert s.at(0) == 0.0 and abs(s.at(5) - 5e-3) < 1e-15 and s.at(10) == 1e-2
    assert abs(s.at(60) - (1e-3 + 0.5 * 9e-3)) < 1e-12           # half way down the cosine
    assert abs(s.at(110) - 1e-3) < 1e-12 and s.at(500) == 1e-3
    assert abs(Schedule(1e-2, 1e-3, 10, 110, "linear").at(35) - (1e-3 + 0.75 * 9e-3)) < 1e-12
    assert Schedule(1e-2, 1e-3, 10, 110, "constant").at(10 ** 6) == 1e-2
    for bad in (dict(peak=1e-3, floor=1e-2), dict(warmup_steps=200), dict(style="exponential")):
        with pytest.raises(ValueError):
            Schedule(**{**dict(peak=1e-2, floor=1e-3, warmup_steps=10, decay_steps=110, style="cosine"), **bad})
    opt = Opt()
    sched = AnnealingLR(opt, 1e-2, 1e-3, 10, 110, "cosine")
    assert opt.lr == 0.0
    sched.step(60)
    assert math.isclose(opt.lr, s.at(60))
    saved = sched.state_dict()
    assert set(saved) == {"max_lr", "min_lr", "warmup_steps", "decay_steps", "decay_style", "num_steps"}
    # checkpoint values win by default; the counter is restored
    other = AnnealingLR(Opt(), 5e-3, 1e-4, 1, 50, "linear")
    other.load_state_dict(saved)
    assert other.max_lr == 1e-2 and other.decay_style == "cosine" and other.num_steps == 60
    # neither flag: a differing value is an error; override: the command line wins, the counter still loads
    strict = AnnealingLR(Opt(), 5e-3, 1e-4, 1, 50, "linear", use_checkpoint_lr_scheduler=False)
    with pytest.raises(ValueError, match="do not match"):
        strict.load_state_dict(saved)
    mine = AnnealingLR(Opt(), 5e-3, 1e-4, 1, 50, "linear", use_checkpoint_lr_scheduler=False, override_lr_scheduler=True)
    mine.load_state_dict(saved)
    assert mine.max_lr == 5e-3 and mine.num_steps == 60
