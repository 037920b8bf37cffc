"""Mixed-precision optimizer over the flat buffers of a stage.

Semantics of the reference's `Float16OptimizerWithFloat16Params` (eth/runtime/megatron/optimizer/
optimizer.py:303-357 master copies, :388-531 step): gradients accumulated in `main_grad` are
unscaled, checked for non-finite values (agreed across the world), the global L2 norm is computed
with each logical element counted once and clipped, AdamW runs on fp32 master weights, and the
16-bit model weights are refreshed. Here that whole sequence is:

    grad_norm_sq over the owned ranges of the flat gradient buffer   (few launches)
    one all-reduce of the 2-float control block [sum of squares, found_inf] over the world
    fused_adam over the weight-decayed region and over the no-decay region (2 launches) which
    unscales, clips by the control block, updates master/moments and writes the 16-bit weights,
    skipping everything when found_inf is set.

Weight decay applies to GEMM / embedding weights only, not to LayerNorm parameters or biases
(reference: optimizer/__init__.py:37-58).
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from ..ops import native


DEVICE_FAULT_MARK = 1024.0   # added to the overflow flag by a rank whose device status word is set


class FlatMixedPrecisionAdam:
    def __init__(self, stage, lr=1.5e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, clip_grad=1.0,
                 grad_scaler=None, owned_ranges: Optional[Sequence[Tuple[int, int]]] = None,
                 world_all_reduce: Optional[Callable[[torch.Tensor], None]] = None, adamw: bool = True,
                 log_num_zeros: bool = False):
        self.stage = stage
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.clip_grad = clip_grad
        self.grad_scaler = grad_scaler
        self.adamw = adamw
        self.world_all_reduce = world_all_reduce
        dev = stage.param_buf.device
        n = stage.total_numel
        self.fp32_params = stage.param_buf.dtype == torch.float32
        self.master = stage.param_buf if self.fp32_params else stage.param_buf.float()
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        # [sum of squares of raw grads, found_inf, raw-to-true gradient factor, spare]
        self.ctrl = torch.zeros(4, dtype=torch.float32, device=dev)
        self.device_grad_factor = False   # True: kernels read ctrl[2] instead of a host float
        self.step_count = 0
        self.owned_ranges = list(owned_ranges) if owned_ranges is not None else [(0, n)]
        self.last_grad_norm = None
        self.last_found_inf = False
        self.last_device_fault = False   # some rank's status word was set when the last step ran

    # -- bookkeeping used by checkpointing and state synchronisation
    def set_lr(self, lr: float) -> None:
        self.lr = lr

    def set_owned_ranges(self, ranges: Sequence[Tuple[int, int]]) -> None:
        self.owned_ranges = coalesce_ranges(ranges)

    def state_for_model_parameter(self, param: torch.Tensor):
        """Views of (master, exp_avg, exp_avg_sq) with the parameter's shape."""
        off = param.storage_offset()
        n = param.numel()
        view = lambda buf: buf[off:off + n].view(param.shape)  # noqa: E731
        out = {"exp_avg": view(self.exp_avg), "exp_avg_sq": view(self.exp_avg_sq)}
        if not self.fp32_params:
            out["master"] = view(self.master)
        return out

    def zero_grad(self) -> None:
        self.stage.zero_grad_buffer()

    def reload_model_params(self) -> None:
        if not self.fp32_params:
            self.master.copy_(self.stage.param_buf.float())

    # -- the step
    def compute_norm_and_inf(self) -> None:
        """ctrl[0] = sum of squares of owned (still loss-scaled) gradients; ctrl[1] = non-finite flag."""
        g = self.stage.grad_buf
        self.ctrl[:2].zero_()
        for off, n in self.owned_ranges:
            if n <= 0:
                continue
            if g.is_cuda:
                native.lib().grad_norm_sq(g[off:off + n], 1.0, self.ctrl)
            else:
                v = g[off:off + n].float()
                self.ctrl[0] += (v * v).sum()
                if not torch.isfinite(v).all():
                    self.ctrl[1] = 1.0
        if g.is_cuda:
            # A bounded device wait that ran out on any rank (status word != 0) left stale or partial
            # data behind: fold it into the overflow flag, so every rank skips this update, with a
            # magnitude the host can tell from a plain overflow.
            self.ctrl[1:2].add_((native.status(g.device) != 0).to(torch.float32), alpha=DEVICE_FAULT_MARK)
        if self.world_all_reduce is not None:
            self.world_all_reduce(self.ctrl[:2])

    def set_grad_factor(self, normalization) -> None:
        """ctrl[2] = normalization / loss_scale, computed on the device (`normalization` may be a
        device scalar such as nominal_scale / global_loss_weight)."""
        scale = self.grad_scaler.value() if self.grad_scaler is not None else 1.0
        if isinstance(normalization, torch.Tensor):
            self.ctrl[2:3].copy_((normalization.float() / scale).reshape(1))
        else:
            self.ctrl[2] = float(normalization) / scale
        self.device_grad_factor = True

    def step(self, sync: bool = True):
        """Returns (update_successful, grad_norm, num_zeros). With sync=False nothing is read back:
        the kernels themselves skip the update on overflow, and the returned values are None."""
        scaler = self.grad_scaler
        inv_scale = scaler.inv_scale if scaler is not None else 1.0
        self.compute_norm_and_inf()
        found_inf, norm = False, None
        if sync:
            host = self.ctrl[:3].tolist()
            if self.device_grad_factor:
                inv_scale = host[2]
            found_inf = host[1] > 0 or not math.isfinite(host[0])
            self.last_device_fault = host[1] >= DEVICE_FAULT_MARK
            norm = math.sqrt(host[0]) * inv_scale if not found_inf else float("nan")
            self.last_grad_norm, self.last_found_inf = norm, found_inf
            if scaler is not None and not self.last_device_fault:
                scaler.update(found_inf)
            if found_inf:
                return False, None, None
        self.step_count += 1
        self._apply(inv_scale)
        return True, norm, None

    def _apply(self, inv_scale: float) -> None:
        st = self.stage
        regions = [(0, st.decay_numel, self.weight_decay), (st.decay_numel, st.total_numel - st.decay_numel, 0.0)]
        b1, b2 = self.betas
        for off, n, wd in regions:
            if n <= 0:
                continue
            sl = slice(off, off + n)
            if st.param_buf.is_cuda:
                native.lib().fused_adam(st.param_buf[sl], self.master[sl], st.grad_buf[sl], self.exp_avg[sl],
                                        self.exp_avg_sq[sl], self.ctrl, self.lr, b1, b2, self.eps, wd,
                                        self.step_count, inv_scale, self.clip_grad, self.adamw,
                                        self.device_grad_factor)
            else:
                self._apply_reference(sl, wd, inv_scale)

    def _apply_reference(self, sl, wd, inv_scale):
        st = self.stage
        if float(self.ctrl[1]) != 0.0:
            return
        if self.device_grad_factor:
            inv_scale = float(self.ctrl[2])
        clip = 1.0
        if self.clip_grad > 0:
            norm = math.sqrt(float(self.ctrl[0])) * inv_scale
            clip = min(1.0, self.clip_grad / (norm + 1.0e-6))
        b1, b2 = self.betas
        g = st.grad_buf[sl].float() * (inv_scale * clip)
        p = self.master[sl]
        if not self.adamw:
            g = g + wd * p
        m, v = self.exp_avg[sl], self.exp_avg_sq[sl]
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        bc1 = 1 - b1 ** self.step_count
        bc2 = 1 - b2 ** self.step_count
        denom = v.sqrt() / math.sqrt(bc2) + self.eps
        if self.adamw:
            p.mul_(1 - self.lr * wd)
        p.addcdiv_(m, denom, value=-self.lr / bc1)
        if not self.fp32_params:
            st.param_buf[sl].copy_(p.to(st.param_buf.dtype))

    # -- (de)serialisation
    def state_dict(self):
        return {"step": self.step_count, "master": None if self.fp32_params else self.master,
                "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "grad_scaler": self.grad_scaler.state_dict() if self.grad_scaler is not None else None,
                "lr": self.lr}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        if sd.get("master") is not None and not self.fp32_params:
            self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        if self.grad_scaler is not None and sd.get("grad_scaler") is not None:
            self.grad_scaler.load_state_dict(sd["grad_scaler"])


def coalesce_ranges(ranges: Sequence[Tuple[int, int]]) -> List[Tuple[int, int]]:
    """Merge (offset, numel) ranges that touch or are separated only by alignment padding (< 128)."""
    out: List[List[int]] = []
    for off, n in sorted(r for r in ranges if r[1] > 0):
        if out and off - (out[-1][0] + out[-1][1]) < 128 and off >= out[-1][0] + out[-1][1]:
            out[-1][1] = off + n - out[-1][0]
        else:
            out.append([off, n])
    return [(a, b) for a, b in out]


def get_optimizer(stage, args, grad_scaler=None, **kw):
    """Factory mirroring the reference's flag surface (optimizer/__init__.py:61-81): adam or sgd."""
    name = getattr(args, "optimizer", "adam")
    if name == "adam":
        return FlatMixedPrecisionAdam(stage, lr=args.lr, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_eps,
                                      weight_decay=args.weight_decay, clip_grad=args.clip_grad,
                                      grad_scaler=grad_scaler, **kw)
    if name == "sgd":
        from .sgd import FlatSGD
        return FlatSGD(stage, lr=args.lr, momentum=getattr(args, "sgd_momentum", 0.9),
                       weight_decay=args.weight_decay, clip_grad=args.clip_grad, grad_scaler=grad_scaler, **kw)
    raise ValueError(f"{name} optimizer is not supported")
