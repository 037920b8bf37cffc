"""Momentum SGD over the flat buffers of a stage (the `--optimizer sgd` choice).

Same wrapper semantics as the Adam path (unscale, agreed overflow skip, global-norm clip on
elements counted once, fp32 master weights, 16-bit refresh); the update is torch.optim.SGD's:
    g <- g + wd * p ;  buf <- momentum * buf + g ;  p <- p - lr * buf
(reference: eth/runtime/megatron/optimizer/__init__.py:70-75 picks torch.optim.SGD under the same
mixed-precision wrapper). It is a handful of flat element-wise passes, not a fused kernel: SGD is
not on any benchmarked path.
"""
from __future__ import annotations


import torch

from .optimizer import FlatMixedPrecisionAdam


class FlatSGD(FlatMixedPrecisionAdam):
    def __init__(self, stage, lr=1.5e-4, momentum=0.9, weight_decay=0.01, clip_grad=1.0, grad_scaler=None, **kw):
        super().__init__(stage, lr=lr, weight_decay=weight_decay, clip_grad=clip_grad, grad_scaler=grad_scaler, **kw)
        self.momentum = momentum
        self.momentum_buf = self.exp_avg          # one state buffer; reuse the allocation
        self.exp_avg_sq = self.exp_avg_sq[:0]     # unused by SGD

    def _apply(self, inv_scale: float) -> None:
        st = self.stage
        # device-side factors so that the async (no host read) mode works as for Adam
        ctrl = self.ctrl
        factor = ctrl[2] if self.device_grad_factor else torch.full_like(ctrl[2], inv_scale)
        ok = (ctrl[1] == 0) & torch.isfinite(ctrl[0])
        clip = torch.ones_like(factor)
        if self.clip_grad > 0:
            norm = ctrl[0].clamp_min(0).sqrt() * factor
            clip = torch.clamp(self.clip_grad / (norm + 1.0e-6), max=1.0)
        mult = torch.where(ok, factor * clip, torch.zeros_like(factor))
        lr = torch.where(ok, torch.full_like(factor, self.lr), torch.zeros_like(factor))
        keep = torch.where(ok, torch.full_like(factor, self.momentum), torch.ones_like(factor))
        regions = [(0, st.decay_numel, self.weight_decay), (st.decay_numel, st.total_numel - st.decay_numel, 0.0)]
        first = self.step_count == 1
        for off, n, wd in regions:
            if n <= 0:
                continue
            sl = slice(off, off + n)
            p, buf = self.master[sl], self.momentum_buf[sl]
            g = st.grad_buf[sl].float() * mult
            g = torch.nan_to_num(g, nan=0.0, posinf=0.0, neginf=0.0)
            if wd:
                g = g + wd * p * (mult != 0)
            if first:
                buf.copy_(torch.where(ok, g, buf))
            else:
                buf.mul_(keep).add_(g)
            p.sub_(buf * lr)
            if not self.fp32_params:
                st.param_buf[sl].copy_(p.to(st.param_buf.dtype))

    def state_dict(self):
        sd = super().state_dict()
        sd["momentum_buffer"] = sd.pop("exp_avg")
        sd.pop("exp_avg_sq", None)
        return sd

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        if sd.get("master") is not None and not self.fp32_params:
            self.master.copy_(sd["master"])
        self.momentum_buf.copy_(sd["momentum_buffer"])
        if self.grad_scaler is not None and sd.get("grad_scaler") is not None:
            self.grad_scaler.load_state_dict(sd["grad_scaler"])
