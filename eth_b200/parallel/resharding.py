"""Intra-stage resharding: moving a tensor from one `{R, V, dims}` placement to another.

`plan_reshard(src, dst)` picks the collective that turns placement `src` into `dst`:
    R  -> dim   split            (replicas each keep a slice; no communication)
    V  -> R     all-reduce       (partial sums become replicas)
    V  -> dim   reduce-scatter
    dim -> R    all-gather
    dim -> dim  all-to-all
with the group size = ratio of the changing factor, and `apply_reshard` runs it on a rank list
through torch.distributed. The backward of each primitive is its dual (`DUAL`), so explicit
backward code calls `apply_reshard` with the dual step. Reference: eth/runtime/megatron/mpu/
mappings.py:149-210 primitives on rank lists, :212-303 autograd duals, :381-467 the adapter;
the search uses the same planner to cost resharding (eth/searching/cost_model.py:52-118).

Public configs keep TP/DP/algo constant inside a stage (the normalizer enforces it), so the
stage program does not call this; it serves per-op layouts in profiling and search.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

DUAL = {"split": "all_gather", "all_gather": "split", "all_reduce": "identity", "identity": "all_reduce",
        "reduce_scatter": "all_gather", "all_to_all": "all_to_all"}


@dataclass(frozen=True)
class ReshardStep:
    primitive: str          # split | all_reduce | reduce_scatter | all_gather | all_to_all | identity
    group_size: int
    src_dim: Optional[int] = None   # dim that is gathered / exchanged away
    dst_dim: Optional[int] = None   # dim that gets split

    def dual(self) -> "ReshardStep":
        p = DUAL[self.primitive]
        if self.primitive == "split":
            return ReshardStep(p, self.group_size, src_dim=self.dst_dim)
        if self.primitive == "all_gather":
            return ReshardStep(p, self.group_size, dst_dim=self.src_dim)
        if self.primitive == "reduce_scatter":
            return ReshardStep(p, self.group_size, src_dim=self.dst_dim)
        if self.primitive == "all_to_all":
            return ReshardStep(p, self.group_size, src_dim=self.dst_dim, dst_dim=self.src_dim)
        return ReshardStep(p, self.group_size)


def spec_size(spec) -> int:
    n = spec["R"] * spec["V"]
    for d in spec["dims"]:
        n *= d
    return n


def identical_spec(a, b) -> bool:
    if not a and not b:
        return True
    return a["R"] == b["R"] and a["V"] == b["V"] and list(a["dims"]) == list(b["dims"])


def plan_reshard(src, dst) -> ReshardStep:
    if not dst or identical_spec(src, dst):
        return ReshardStep("identity", 1)
    if spec_size(src) != spec_size(dst):
        raise ValueError(f"placements cover different numbers of devices: {src} vs {dst}")
    dims = range(len(src["dims"]))
    if src["R"] > dst["R"]:
        for d in dims:
            if src["dims"][d] < dst["dims"][d]:
                if src["R"] % dst["R"]:
                    raise ValueError("replica count must divide")
                return ReshardStep("split", src["R"] // dst["R"], dst_dim=d)
    elif src["V"] > dst["V"]:
        if src["V"] % dst["V"]:
            raise ValueError("partial-sum count must divide")
        if src["R"] < dst["R"]:
            return ReshardStep("all_reduce", src["V"] // dst["V"])
        for d in dims:
            if src["dims"][d] < dst["dims"][d]:
                return ReshardStep("reduce_scatter", src["V"] // dst["V"], dst_dim=d)
    else:
        for s in dims:
            if src["dims"][s] > dst["dims"][s]:
                if src["dims"][s] % dst["dims"][s]:
                    raise ValueError("split factor must divide")
                n = src["dims"][s] // dst["dims"][s]
                if src["R"] < dst["R"]:
                    return ReshardStep("all_gather", n, src_dim=s)
                for d in dims:
                    if d != s and src["dims"][d] < dst["dims"][d]:
                        return ReshardStep("all_to_all", n, src_dim=s, dst_dim=d)
    raise RuntimeError(f"No communication pattern found. input_spec: {src}\nrequired_spec: {dst}")


def reshard_bytes(step: ReshardStep, tensor_bytes: float) -> float:
    """Bytes each rank sends for `step` on a local tensor of `tensor_bytes` (for cost models)."""
    n = step.group_size
    if step.primitive in ("identity", "split") or n <= 1:
        return 0.0
    if step.primitive == "all_reduce":
        return 2.0 * (n - 1) / n * tensor_bytes
    return (n - 1) / n * tensor_bytes


def apply_reshard(x: torch.Tensor, step: ReshardStep, group=None, group_rank: Optional[int] = None) -> torch.Tensor:
    """Run one step on `group` (its size must equal step.group_size)."""
    n = step.group_size
    if step.primitive == "identity" or n <= 1:
        return x
    if group_rank is None:
        group_rank = dist.get_rank(group)
    if step.primitive == "split":
        return x.chunk(n, dim=step.dst_dim)[group_rank].contiguous()
    if step.primitive == "all_reduce":
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y
    if step.primitive == "all_gather":
        parts = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=step.src_dim)
    if step.primitive == "reduce_scatter":
        chunks = [c.contiguous() for c in x.chunk(n, dim=step.dst_dim)]
        out = torch.empty_like(chunks[0])
        if dist.get_backend(group) == "gloo":
            y = x.clone()
            dist.all_reduce(y, group=group)
            return y.chunk(n, dim=step.dst_dim)[group_rank].contiguous()
        dist.reduce_scatter(out, chunks, group=group)
        return out
    if step.primitive == "all_to_all":
        send = [c.contiguous() for c in x.chunk(n, dim=step.dst_dim)]
        recv = [torch.empty_like(send[0]) for _ in range(n)]
        if dist.get_backend(group) == "gloo":
            gathered = [torch.empty_like(x) for _ in range(n)]
            dist.all_gather(gathered, x.contiguous(), group=group)
            recv = [g.chunk(n, dim=step.dst_dim)[group_rank] for g in gathered]
        else:
            dist.all_to_all(recv, send, group=group)
        return torch.cat(recv, dim=step.src_dim)
    raise ValueError(f"unknown primitive {step.primitive!r}")


# ------------------------------------------------------------------------------------------
# autograd adapters (library use; the stage program calls `apply_reshard` with explicit duals)
# ------------------------------------------------------------------------------------------
class _Reshard(torch.autograd.Function):
    """One placement change whose backward is its dual, whatever the primitive: the table `DUAL`
    replaces one autograd class per primitive (reference: mpu/mappings.py:212-303)."""

    @staticmethod
    def forward(ctx, x, step, group, group_rank):
        ctx.step, ctx.group, ctx.group_rank = step, group, group_rank
        return apply_reshard(x, step, group, group_rank)

    @staticmethod
    def backward(ctx, grad):
        return apply_reshard(grad.contiguous(), ctx.step.dual(), ctx.group, ctx.group_rank), None, None, None


def reshard(x: torch.Tensor, step: ReshardStep, group=None, group_rank: Optional[int] = None) -> torch.Tensor:
    """`apply_reshard` that autograd can differentiate."""
    if step.primitive == "identity" and step.group_size <= 1:
        return x
    return _Reshard.apply(x, step, group, group_rank)


def tensor_adapter(x: torch.Tensor, src_spec, dst_spec, group=None, group_rank: Optional[int] = None) -> torch.Tensor:
    """Move `x` from placement `src_spec` to `dst_spec` (reference: mpu/mappings.py:381-467)."""
    return reshard(x, plan_reshard(src_spec, dst_spec), group, group_rank)


def copy_to_region(x, group=None):
    """Identity forward, all-reduce backward: the input of a column-parallel layer."""
    n = dist.get_world_size(group)
    return reshard(x, ReshardStep("identity", n), group)


def reduce_from_region(x, group=None):
    """All-reduce forward, identity backward: the output of a row-parallel layer."""
    return reshard(x, ReshardStep("all_reduce", dist.get_world_size(group)), group)


def scatter_to_region(x, group=None, dim: int = -1):
    """Keep this rank's slice along `dim` forward, all-gather backward."""
    return reshard(x, ReshardStep("split", dist.get_world_size(group), dst_dim=dim % x.dim()), group)


def gather_from_region(x, group=None, dim: int = -1):
    """All-gather along `dim` forward, slice backward."""
    return reshard(x, ReshardStep("all_gather", dist.get_world_size(group), src_dim=dim % x.dim()), group)
