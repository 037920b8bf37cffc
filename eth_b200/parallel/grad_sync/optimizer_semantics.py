"""Canonical parameter consistency, gradient-norm ownership and clipping.

Every fragment has one owner rank (the smallest rank of its group). Quantities that must be
counted once per *logical* element -- the global gradient norm, the zero count -- are computed
from owned fragments only and summed over the world; operations that must agree across all
holders of a logical element -- initial parameters, optimizer moments after a checkpoint load --
are broadcast fragment by fragment from the owner
(reference: eth/runtime/megatron/grad_sync/optimizer_semantics.py:258-279 parameters,
:318-358 optimizer state, :537-604 norm / clip / zero count).

Tied weights need no extra path here: both copies of a tied weight are holders of the same
fragments (see planner), so the fragment broadcasts and the fragment all-reduce keep them equal.
"""
from __future__ import annotations

import math

import torch


class CanonicalOptimizerSemantics:
    def __init__(self, plan, global_rank, local_descriptors, local_runtime_bindings, control_device="cpu"):
        self.plan = plan
        self.global_rank = global_rank
        self.control_device = torch.device(control_device)
        self._fragments = {f.fragment_id: f for f in plan.canonical_fragments}
        self._groups = {g.process_group_id: g for g in plan.process_groups}
        self._descriptors = self._index(local_descriptors, "descriptor")
        self._bindings = self._index(local_runtime_bindings, "runtime binding")
        self._by_param = {id(b.parameter): b.logical_param_id for b in local_runtime_bindings}
        self._opt_grads = {}
        self._specs = {b.fragment_id: b for r, bs in plan.local_fragment_bindings_by_rank if r == global_rank
                       for b in bs}

    @staticmethod
    def _index(items, kind):
        out = {}
        for it in items:
            if it.logical_param_id in out:
                raise ValueError(f"duplicate {kind} for logical_param_id {it.logical_param_id}")
            out[it.logical_param_id] = it
        return out

    # -- gradient tensors the optimizer actually steps on (fp32 copies of main_grad, if any)
    def bind_optimizer_gradient(self, model_parameter, gradient):
        lid = self._by_param.get(id(model_parameter))
        if lid is None:
            raise ValueError("model parameter has no canonical gradient binding")
        if tuple(gradient.shape) != tuple(model_parameter.shape):
            raise ValueError(f"optimizer gradient shape mismatch for {lid}: expected "
                             f"{tuple(model_parameter.shape)}, got {tuple(gradient.shape)}")
        self._opt_grads[lid] = gradient

    def _gradient(self, lid):
        return self._opt_grads.get(lid, self._bindings[lid].main_grad)

    def _views(self, tensor, spec):
        desc = self._descriptors[spec.logical_param_id]
        if not desc.tensor_parallel:
            if len(spec.source_segments) != 1:
                raise ValueError(f"logical_param_id {spec.logical_param_id} replicated binding must have one segment")
            if spec.source_segments[0].flattened_numel != tensor.numel():
                raise ValueError(f"logical_param_id {spec.logical_param_id} replicated source numel mismatch")
            yield tensor
            return
        axis = desc.partition_dim + (tensor.dim() if desc.partition_dim < 0 else 0)
        for seg in spec.source_segments:
            if math.prod(seg.source_shape) != tensor.numel():
                raise ValueError(f"logical_param_id {spec.logical_param_id} source shape mismatch")
            yield tensor.narrow(axis, seg.source_dim_offset, seg.source_dim_length)

    def _gather(self, tensor, spec, frag):
        out = torch.empty(frag.numel, dtype=tensor.dtype, device=tensor.device)
        cur = 0
        for v in self._views(tensor, spec):
            out[cur:cur + v.numel()].copy_(v.reshape(-1))
            cur += v.numel()
        if cur != frag.numel:
            raise ValueError(f"fragment {frag.fragment_id} logical_param_id {spec.logical_param_id} "
                             f"packed {cur}, expected {frag.numel}")
        return out

    def _scatter(self, tensor, spec, frag, payload):
        cur = 0
        for v in self._views(tensor, spec):
            v.copy_(payload[cur:cur + v.numel()].view(v.shape))
            cur += v.numel()
        if cur != frag.numel:
            raise ValueError(f"fragment {frag.fragment_id} unpacked {cur}, expected {frag.numel}")

    def _my_fragments(self):
        for frag in self.plan.canonical_fragments:
            spec = self._specs.get(frag.fragment_id)
            if spec is not None:
                yield frag, spec, self._bindings[spec.logical_param_id], self._groups[frag.process_group_id]

    # -- broadcasts: broadcast(payload, source_rank, process_group_id, group_ranks, tag, current_rank)
    def synchronize_parameters(self, broadcast):
        for frag, spec, rt, group in self._my_fragments():
            payload = self._gather(rt.parameter.data, spec, frag)
            broadcast(payload, min(group.ranks), frag.process_group_id, group.ranks, frag.fragment_id, self.global_rank)
            self._scatter(rt.parameter.data, spec, frag, payload)

    def synchronize_shared_root_gradients(self, broadcast):
        """Tied weights are holders of common fragments here, so their gradients are already equal
        after the fragment all-reduce. Kept so callers written against the reference flow work."""
        return None

    def optimizer_state_manifest_for_group(self, process_group_id, state_for_parameter):
        rows = []
        for frag, spec, rt, _ in self._my_fragments():
            if frag.process_group_id != process_group_id:
                continue
            state = state_for_parameter(rt.parameter)
            entry = []
            for name in sorted(state):
                t = state[name]
                if not isinstance(t, torch.Tensor):
                    continue
                if tuple(t.shape) == tuple(rt.parameter.shape):
                    kind = "parameter"
                elif t.numel() == 1:
                    kind = "scalar"
                else:
                    raise ValueError(f"optimizer state shape mismatch for {spec.logical_param_id}.{name}: {tuple(t.shape)}")
                entry.append((name, kind, str(t.dtype)))
            rows.append((frag.fragment_id, tuple(entry)))
        return tuple(rows)

    def synchronize_optimizer_state(self, state_for_parameter, broadcast):
        for frag, spec, rt, group in self._my_fragments():
            state = state_for_parameter(rt.parameter)
            src = min(group.ranks)
            for name in sorted(state):
                t = state[name]
                if not isinstance(t, torch.Tensor):
                    continue
                if tuple(t.shape) == tuple(rt.parameter.shape):
                    payload = self._gather(t, spec, frag)
                    broadcast(payload, src, frag.process_group_id, group.ranks, f"{frag.fragment_id}:{name}", self.global_rank)
                    self._scatter(t, spec, frag, payload)
                elif t.numel() == 1:
                    payload = t.reshape(-1).clone()
                    broadcast(payload, src, frag.process_group_id, group.ranks, f"{frag.fragment_id}:{name}", self.global_rank)
                    t.copy_(payload.view(t.shape))
                else:
                    raise ValueError(f"optimizer state shape mismatch for {spec.logical_param_id}.{name}: {tuple(t.shape)}")

    # -- norm ownership
    def owned_gradient_views(self):
        for frag in self.plan.canonical_fragments:
            if not frag.include_in_optimizer_norm or frag.norm_owner_rank != self.global_rank:
                continue
            spec = self._specs.get(frag.fragment_id)
            if spec is None:
                raise ValueError(f"norm owner rank {self.global_rank} is missing binding for fragment {frag.fragment_id}")
            yield from self._views(self._gradient(spec.logical_param_id), spec)

    def all_local_gradients(self):
        seen = set()
        for lid in sorted(self._bindings):
            g = self._gradient(lid)
            if id(g) not in seen:
                seen.add(id(g))
                yield g

    def owned_norm_sq(self, inv_scale=1.0):
        """Device scalar: sum of squares of the gradient elements this rank owns."""
        total = None
        for v in self.owned_gradient_views():
            s = (v.detach().float() * inv_scale).pow(2).sum()
            total = s if total is None else total + s
        if total is None:
            total = torch.zeros((), dtype=torch.float32, device=self.control_device)
        return total

    def clip_grad_norm(self, max_norm, norm_type, all_reduce_sum, all_reduce_max):
        max_norm, norm_type = float(max_norm), float(norm_type)
        stat = torch.zeros((), dtype=torch.float32, device=self.control_device)
        if norm_type == float("inf"):
            for v in self.owned_gradient_views():
                if v.numel():
                    stat.copy_(torch.maximum(stat, v.detach().abs().max().float().to(stat.device)))
            all_reduce_max(stat, "inf_norm")
            total = float(stat.item())
        elif norm_type == 2.0:
            for v in self.owned_gradient_views():
                stat.add_(v.detach().float().pow(2).sum().to(stat.device))
            all_reduce_sum(stat, "l2_norm_sq")
            total = math.sqrt(float(stat.item()))
        else:
            raise ValueError(f"unsupported canonical norm type {norm_type}")
        coef = max_norm / (total + 1.0e-6)
        if coef < 1.0:
            for g in self.all_local_gradients():
                g.mul_(coef)
        return total

    def count_zeros(self, all_reduce_sum):
        total = torch.zeros((), dtype=torch.float32, device=self.control_device)
        for v in self.owned_gradient_views():
            total.add_((v.numel() - torch.count_nonzero(v)).to(total.device))
        all_reduce_sum(total, "zero_count")
        return float(total.item())
