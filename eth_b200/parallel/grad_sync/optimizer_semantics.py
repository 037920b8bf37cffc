"""Canonical parameter consistency, gradient-norm ownership and clipping.

Every fragment has one owner rank (the smallest rank of its group). Two kinds of operation build
on that:

  * "make all holders equal": the owner's values of a fragment are broadcast to the other holders.
    Used for the initial parameters and, after a checkpoint load, for parameters and optimizer
    moments. One routine (`_replicate`) does it for any tensor shaped like the parameter.
  * "count once": the global gradient norm and the zero count take each logical element from its
    owner only and are summed over the world.

(reference: eth/runtime/megatron/grad_sync/optimizer_semantics.py:258-279 parameters, :318-358
optimizer state, :537-604 norm / clip / zero count). Tied weights need no extra path here: both
copies of a tied weight are holders of the same fragments (see planner), so the fragment
broadcasts and the fragment all-reduce keep them equal.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Iterator, List, Tuple

import torch


@dataclass(frozen=True)
class _BoundFragment:
    """A fragment this rank holds: where it sits in tensors shaped like the local parameter."""
    fragment: object
    logical_id: str
    group_ranks: Tuple[int, ...]
    axis: int                                    # -1: the whole tensor (replicated parameter)
    pieces: Tuple[Tuple[int, int], ...]          # (offset, length) along `axis`
    local_numel: int

    @property
    def owner(self) -> int:
        return min(self.group_ranks)

    def views(self, tensor: torch.Tensor) -> List[torch.Tensor]:
        if tensor.numel() != self.local_numel:
            raise ValueError(f"logical_param_id {self.logical_id} source shape mismatch")
        if self.axis < 0:
            return [tensor]
        return [tensor.narrow(self.axis, off, n) for off, n in self.pieces]

    def read(self, tensor: torch.Tensor) -> torch.Tensor:
        flat = torch.cat([v.reshape(-1) for v in self.views(tensor)])
        if flat.numel() != self.fragment.numel:
            raise ValueError(f"fragment {self.fragment.fragment_id} logical_param_id {self.logical_id} "
                             f"packed {flat.numel()}, expected {self.fragment.numel}")
        return flat

    def write(self, tensor: torch.Tensor, flat: torch.Tensor) -> None:
        at = 0
        for v in self.views(tensor):
            v.copy_(flat[at:at + v.numel()].view(v.shape))
            at += v.numel()


def _unique_by_logical_id(items, what):
    table = {}
    for it in items:
        if it.logical_param_id in table:
            raise ValueError(f"duplicate {what} for logical_param_id {it.logical_param_id}")
        table[it.logical_param_id] = it
    return table


def _parameter_shaped_state(state: dict, parameter, logical_id) -> Iterator[Tuple[str, torch.Tensor, str]]:
    """(name, tensor, kind) of the tensor entries of one parameter's optimizer state, by name."""
    for name in sorted(state):
        t = state[name]
        if not isinstance(t, torch.Tensor):
            continue
        if tuple(t.shape) == tuple(parameter.shape):
            yield name, t, "parameter"
        elif t.numel() == 1:
            yield name, t, "scalar"
        else:
            raise ValueError(f"optimizer state shape mismatch for {logical_id}.{name}: {tuple(t.shape)}")


class CanonicalOptimizerSemantics:
    def __init__(self, plan, global_rank, local_descriptors, local_runtime_bindings, control_device="cpu"):
        self.plan, self.global_rank = plan, global_rank
        self.control_device = torch.device(control_device)
        descriptors = _unique_by_logical_id(local_descriptors, "descriptor")
        self._bindings = _unique_by_logical_id(local_runtime_bindings, "runtime binding")
        self._logical_id_of = {id(b.parameter): b.logical_param_id for b in local_runtime_bindings}
        self._step_gradients = {}       # logical id -> the tensor the optimizer steps on, if not main_grad
        ranks_of = {g.process_group_id: g.ranks for g in plan.process_groups}
        mine = {b.fragment_id: b for b in dict(plan.local_fragment_bindings_by_rank).get(global_rank, ())}
        self._bound: List[_BoundFragment] = []
        for frag in plan.canonical_fragments:            # plan order = the order every holder walks
            spec = mine.get(frag.fragment_id)
            if spec is None:
                continue
            desc = descriptors[spec.logical_param_id]
            local_numel = math.prod(spec.source_segments[0].source_shape) if spec.source_segments[0].source_shape else 1
            if desc.tensor_parallel:
                ndim = len(desc.local_shape)
                axis = desc.partition_dim + ndim if desc.partition_dim < 0 else desc.partition_dim
                pieces = tuple((s.source_dim_offset, s.source_dim_length) for s in spec.source_segments)
            else:
                if len(spec.source_segments) != 1:
                    raise ValueError(f"logical_param_id {spec.logical_param_id} replicated binding must have one segment")
                axis, pieces = -1, ()
            self._bound.append(_BoundFragment(frag, spec.logical_param_id, ranks_of[frag.process_group_id], axis,
                                              pieces, local_numel))

    # ------------------------------------------------------------------ which gradient tensor counts
    def bind_optimizer_gradient(self, model_parameter, gradient):
        """Tell the semantics layer that the optimizer steps on `gradient` (e.g. an fp32 copy) rather
        than on the parameter's `main_grad`."""
        lid = self._logical_id_of.get(id(model_parameter))
        if lid is None:
            raise ValueError("model parameter has no canonical gradient binding")
        if tuple(gradient.shape) != tuple(model_parameter.shape):
            raise ValueError(f"optimizer gradient shape mismatch for {lid}: expected "
                             f"{tuple(model_parameter.shape)}, got {tuple(gradient.shape)}")
        self._step_gradients[lid] = gradient

    def _gradient(self, logical_id):
        return self._step_gradients.get(logical_id, self._bindings[logical_id].main_grad)

    # ------------------------------------------------------------------ make all holders equal
    # broadcast(payload, source_rank, process_group_id, group_ranks, tag, current_rank)
    def _replicate(self, tensors_of: Callable, broadcast) -> None:
        """For every bound fragment, in plan order, and every (tag, tensor) that `tensors_of(binding)`
        yields: overwrite this rank's slice of the tensor with the owner's."""
        for bf in self._bound:
            for tag, tensor, kind in tensors_of(self._bindings[bf.logical_id], bf):
                label = bf.fragment.fragment_id + tag
                if kind == "scalar":
                    box = tensor.reshape(-1).clone()
                    broadcast(box, bf.owner, bf.fragment.process_group_id, bf.group_ranks, label, self.global_rank)
                    tensor.copy_(box.view(tensor.shape))
                else:
                    flat = bf.read(tensor)
                    broadcast(flat, bf.owner, bf.fragment.process_group_id, bf.group_ranks, label, self.global_rank)
                    bf.write(tensor, flat)

    def synchronize_parameters(self, broadcast):
        self._replicate(lambda binding, bf: [("", binding.parameter.data, "parameter")], broadcast)

    def synchronize_shared_root_gradients(self, broadcast):
        """Tied weights are holders of common fragments here, so their gradients are already equal
        after the fragment all-reduce. Kept so callers written against the reference flow work."""
        return None

    def synchronize_optimizer_state(self, state_for_parameter, broadcast):
        def moments(binding, bf):
            state = state_for_parameter(binding.parameter)
            return [(":" + name, t, kind) for name, t, kind in _parameter_shaped_state(state, binding.parameter, bf.logical_id)]
        self._replicate(moments, broadcast)

    def optimizer_state_manifest_for_group(self, process_group_id, state_for_parameter):
        """What the members of a group compare before optimizer state is replicated."""
        rows = []
        for bf in self._bound:
            if bf.fragment.process_group_id != process_group_id:
                continue
            parameter = self._bindings[bf.logical_id].parameter
            entries = tuple((name, kind, str(t.dtype)) for name, t, kind in
                            _parameter_shaped_state(state_for_parameter(parameter), parameter, bf.logical_id))
            rows.append((bf.fragment.fragment_id, entries))
        return tuple(rows)

    # ------------------------------------------------------------------ count once
    def owned_gradient_views(self):
        """Views of the gradient elements whose norm contribution this rank is responsible for."""
        have = {bf.fragment.fragment_id for bf in self._bound}
        for frag in self.plan.canonical_fragments:
            if frag.include_in_optimizer_norm and frag.norm_owner_rank == self.global_rank and frag.fragment_id not in have:
                raise ValueError(f"norm owner rank {self.global_rank} is missing binding for fragment {frag.fragment_id}")
        for bf in self._bound:
            if bf.fragment.include_in_optimizer_norm and bf.fragment.norm_owner_rank == self.global_rank:
                yield from bf.views(self._gradient(bf.logical_id))

    def all_local_gradients(self):
        seen = set()
        for lid in sorted(self._bindings):
            g = self._gradient(lid)
            if id(g) not in seen:
                seen.add(id(g))
                yield g

    def _zero_scalar(self):
        return torch.zeros((), dtype=torch.float32, device=self.control_device)

    def owned_norm_sq(self, inv_scale=1.0):
        """Device scalar: sum of squares of the gradient elements this rank owns."""
        total = self._zero_scalar()
        for v in self.owned_gradient_views():
            total = total + (v.detach().float() * inv_scale).pow(2).sum().to(total.device)
        return total

    def clip_grad_norm(self, max_norm, norm_type, all_reduce_sum, all_reduce_max):
        """Global norm with every logical element counted once; scales all local gradients."""
        norm_type = float(norm_type)
        acc = self._zero_scalar()
        if norm_type == math.inf:
            for v in self.owned_gradient_views():
                if v.numel():
                    acc = torch.maximum(acc, v.detach().abs().max().float().to(acc.device))
            all_reduce_max(acc, "inf_norm")
            norm = float(acc.item())
        elif norm_type == 2.0:
            acc = self.owned_norm_sq()
            all_reduce_sum(acc, "l2_norm_sq")
            norm = math.sqrt(float(acc.item()))
        else:
            raise ValueError(f"unsupported canonical norm type {norm_type}")
        factor = float(max_norm) / (norm + 1.0e-6)
        if factor < 1.0:
            for g in self.all_local_gradients():
                g.mul_(factor)
        return norm

    def count_zeros(self, all_reduce_sum):
        zeros = self._zero_scalar()
        for v in self.owned_gradient_views():
            zeros = zeros + (v.numel() - torch.count_nonzero(v)).to(zeros.device)
        all_reduce_sum(zeros, "zero_count")
        return float(zeros.item())
