"""Canonical gradient sync without devices: topology, fragment planner, bucket plan, executor with
in-memory collectives, manager agreement checks, optimizer semantics."""
from dataclasses import replace

import pytest
import torch

from eth_b200.contract import config as C
from eth_b200.parallel.grad_sync import buckets as B
from eth_b200.parallel.grad_sync import planner as P
from eth_b200.parallel.grad_sync.descriptors import LocalGradientBinding, SerializableGradientDescriptor
from eth_b200.parallel.grad_sync.executor import GradientBucketExecutor
from eth_b200.parallel.grad_sync.manager import initialize_gradient_sync
from eth_b200.parallel.grad_sync.optimizer_semantics import CanonicalOptimizerSemantics
from eth_b200.parallel.grad_sync.topology import build_canonical_topology


def _topology(pipes):
    return build_canonical_topology(C.normalize_flexpipe_config(C.make_config(pipes)))


def _desc(topo, rank, lid, full, pdim, order=(1, 0, "w"), dtype="float32"):
    f = topo.expected_rank_facts(rank)
    tp, tpr = f["tp_degree"], f["tp_rank"]
    local = list(full)
    if pdim >= 0:
        local[pdim] //= tp
    return SerializableGradientDescriptor(
        logical_param_id=lid, shared_weight_id=None, shared_weight_root=False, logical_region_key=lid,
        semantic_order_key=order, global_rank=rank, model_impl="gpt", op_manifest_hash="m", pipeline_id=f["pipeline_id"],
        stage_id=f["stage_id"], model_chunk_id=0, global_op_index=1, manifest_op_name="op", runtime_op_name="Op",
        relative_parameter_name="weight", stage_global_op_begin=f["global_op_begin"], stage_global_op_end=f["global_op_end"],
        local_tp_degree=tp, local_tp_rank=tpr, local_dp_degree=f["dp_degree"], local_dp_rank=f["dp_rank"], local_cp_degree=1,
        local_cp_rank=0, stage_ranks=f["stage_ranks"], local_tp_group_ranks=f["tp_group_ranks"],
        local_dp_group_ranks=f["dp_group_ranks"], full_shape=tuple(full), local_shape=tuple(local), tensor_parallel=pdim >= 0,
        tp_replica_semantics=None if pdim >= 0 else "identical_duplicate", partition_dim=pdim, partition_stride=1,
        parameter_dtype=dtype, gradient_dtype=dtype, requires_grad=True)


# pipeline 0: one stage TP1 x DP2 (ranks 0, 1); pipeline 1: one stage TP2 x DP1 (ranks 2, 3)
TOPO = _topology([C.make_pipe([43], [1], [2]), C.make_pipe([43], [2], [1])])


def _all_descs():
    out = []
    for r in range(4):
        out.append(_desc(TOPO, r, "gpt.layers.0.col.weight", (8, 4), 0, (1, 0, "a")))
        out.append(_desc(TOPO, r, "gpt.layers.0.row.weight", (4, 8), 1, (1, 0, "b")))
        out.append(_desc(TOPO, r, "gpt.layers.0.ln.weight", (4,), -1, (1, 0, "c")))
    return out


def test_topology_layout():
    s = TOPO.stage(1, 0)
    assert s.stage_ranks == (2, 3) and s.tp_group_ranks_by_coordinate == ((2, 3),) and s.dp_group_ranks_by_coordinate == ((2,), (3,))
    assert TOPO.stage(0, 0).dp_group_ranks_by_coordinate == ((0, 1),)
    assert TOPO.expected_rank_facts(3)["tp_rank"] == 1


def test_fragments_span_pipelines_with_different_tp():
    plan = P.plan_canonical_fragments(_all_descs(), [0, 1])
    col = [f for f in plan.fragments if f.logical_param_id.endswith("col.weight")]
    assert len(col) == 2   # canonical TP degree 2
    groups = {g.process_group_id: g.ranks for g in plan.process_groups}
    assert sorted(groups[f.process_group_id] for f in col) == [(0, 1, 2), (0, 1, 3)]
    ln = [f for f in plan.fragments if f.logical_param_id.endswith("ln.weight")][0]
    assert groups[ln.process_group_id] == (0, 1, 2, 3) and ln.reduction_semantics == "sum_identical_duplicates"
    # the TP=1 holder binds both canonical shards as slices of its one tensor
    b0 = [b for b in plan.bindings_for_rank(0) if b.logical_param_id.endswith("row.weight")]
    assert sorted(s.source_dim_offset for b in b0 for s in b.source_segments) == [0, 4]
    scales = {b.contribution_scale for b in plan.bindings_for_rank(2) if b.logical_param_id.endswith("ln.weight")}
    assert scales == {0.5}
    assert all(f.norm_owner_rank == min(groups[f.process_group_id]) for f in plan.fragments)
    assert plan.fragment_hash == P.plan_canonical_fragments(list(reversed(_all_descs())), [0, 1]).fragment_hash


def test_planner_rejects_inconsistent_holders():
    d = _all_descs()
    with pytest.raises(ValueError, match="missing owner pipeline"):
        P.plan_canonical_fragments([x for x in d if x.pipeline_id == 0], [0, 1])
    bad = [replace(x, full_shape=(8, 5)) if x.global_rank == 3 and x.logical_param_id.endswith("col.weight") else x for x in d]
    with pytest.raises(ValueError, match="shape mismatch"):
        P.plan_canonical_fragments(bad, [0, 1])
    with pytest.raises(ValueError, match="duplicate owner rank"):
        P.plan_canonical_fragments(d + [d[0]], [0, 1])


def test_bucket_modes_and_hashes():
    frag = P.plan_canonical_fragments(_all_descs(), [0, 1])
    tensor = B.build_gradient_sync_plan(frag, "tensor", 1 << 20, "gpt", "m", "t")
    block = B.build_gradient_sync_plan(frag, "block", 1 << 20, "gpt", "m", "t")
    tiny = B.build_gradient_sync_plan(frag, "block", 16, "gpt", "m", "t")
    assert len(tensor.global_bucket_order) == len(frag.fragments)
    assert len(block.global_bucket_order) < len(tensor.global_bucket_order)
    assert all(b.oversized for b in tiny.global_bucket_order if b.exact_bytes > 16)
    assert dict(tensor.exact_payload_bytes_by_rank) == dict(block.exact_payload_bytes_by_rank)
    assert block.padding_payload_bytes == 0 and block.global_plan_hash != tensor.global_plan_hash
    assert block.global_fragment_hash == tensor.global_fragment_hash
    with pytest.raises(ValueError, match="unsupported sync mode"):
        B.build_gradient_sync_plan(frag, "bogus", 16, "gpt", "m", "t")


class World:
    """In-memory world of 4 ranks: runs every rank's executor and sums payloads per group."""

    def __init__(self, mode="block"):
        self.descs = _all_descs()
        frag = P.plan_canonical_fragments(self.descs, [0, 1])
        self.plan = B.build_gradient_sync_plan(frag, mode, 1 << 20, "gpt", "m", "t")
        self.grads = {}
        self.execs = {}
        self.pending = {}
        for r in range(4):
            local = [d for d in self.descs if d.global_rank == r]
            binds = []
            for d in local:
                g = torch.arange(1, 1 + torch.Size(d.local_shape).numel(), dtype=torch.float32).view(d.local_shape) * (r + 1)
                p = torch.zeros(d.local_shape)
                self.grads[(r, d.logical_param_id)] = g
                binds.append(LocalGradientBinding(d.logical_param_id, p, g, g.device))
            reg = B.ProcessGroupRegistry(self.plan.process_groups, lambda ranks: ranks)
            reg.initialize()
            self.execs[r] = GradientBucketExecutor(self.plan, r, local, binds, reg, None)

    def run(self, scale=1.0):
        # lock-step over buckets: pack on all member ranks, sum, unpack
        groups = {g.process_group_id: g.ranks for g in self.plan.process_groups}
        for bucket in self.plan.global_bucket_order:
            ranks = groups[bucket.process_group_id]
            payloads = {}
            for r in ranks:
                ex = self.execs[r]
                payloads[r] = ex.scratch(bucket.grad_dtype)[:bucket.exact_numel]
                ex.pack(bucket, payloads[r])
            total = sum(payloads.values())
            for r in ranks:
                payloads[r].copy_(total)
                self.execs[r].unpack(bucket, payloads[r], scale)


def test_executor_sums_canonical_shards_across_layouts():
    w = World("block")
    before = {k: v.clone() for k, v in w.grads.items()}
    w.run(scale=0.5)
    # column weight (8 x 4): full grads of ranks 0, 1 plus the two TP halves of ranks 2 / 3
    full_p1 = torch.cat([before[(2, "gpt.layers.0.col.weight")], before[(3, "gpt.layers.0.col.weight")]], 0)
    want = 0.5 * (before[(0, "gpt.layers.0.col.weight")] + before[(1, "gpt.layers.0.col.weight")] + full_p1)
    assert torch.allclose(w.grads[(0, "gpt.layers.0.col.weight")], want)
    assert torch.allclose(w.grads[(3, "gpt.layers.0.col.weight")], want[4:])
    # row weight is cut along dim 1
    full_p1 = torch.cat([before[(2, "gpt.layers.0.row.weight")], before[(3, "gpt.layers.0.row.weight")]], 1)
    want = 0.5 * (before[(0, "gpt.layers.0.row.weight")] + before[(1, "gpt.layers.0.row.weight")] + full_p1)
    assert torch.allclose(w.grads[(1, "gpt.layers.0.row.weight")], want)
    assert torch.allclose(w.grads[(2, "gpt.layers.0.row.weight")], want[:, :4])
    # replicated: TP peers contribute half each
    ln = "gpt.layers.0.ln.weight"
    want = 0.5 * (before[(0, ln)] + before[(1, ln)] + 0.5 * before[(2, ln)] + 0.5 * before[(3, ln)])
    for r in range(4):
        assert torch.allclose(w.grads[(r, ln)], want)


def test_tensor_and_block_modes_agree():
    a, b = World("tensor"), World("block")
    a.run()
    b.run()
    for k in a.grads:
        assert torch.equal(a.grads[k], b.grads[k])


def test_norm_counts_every_logical_element_once():
    w = World("block")
    w.run()
    total = 0.0
    for r in range(4):
        local = [d for d in w.descs if d.global_rank == r]
        binds = [LocalGradientBinding(d.logical_param_id, torch.zeros(d.local_shape), w.grads[(r, d.logical_param_id)], "cpu")
                 for d in local]
        sem = CanonicalOptimizerSemantics(w.plan, r, local, binds)
        total += float(sem.owned_norm_sq())
    want = sum(float(w.grads[(0, d.logical_param_id)].pow(2).sum()) for d in w.descs if d.global_rank == 0)
    assert abs(total - want) / want < 1e-6


def test_manager_detects_plan_hash_mismatch():
    descs = _all_descs()
    local = [d for d in descs if d.global_rank == 0]
    binds = [LocalGradientBinding(d.logical_param_id, torch.zeros(d.local_shape), torch.zeros(d.local_shape), "cpu") for d in local]

    def gather(out, obj):
        if isinstance(obj, str):   # plan hash: pretend rank 3 disagrees
            out[:] = [obj, obj, obj, "different"]
        else:
            for r in range(4):
                out[r] = tuple(d for d in descs if d.global_rank == r)

    with pytest.raises(ValueError, match="plan hash mismatch"):
        initialize_gradient_sync(local_descriptors=local, local_runtime_bindings=binds, topology=TOPO, model_impl="gpt",
                                 manifest_hash="m", sync_mode="block", bucket_cap_bytes=1 << 20, global_rank=0,
                                 all_gather_object=gather, all_gather_group_object=lambda o, x, h: o.__setitem__(slice(None), [x] * len(o)),
                                 create_group=lambda ranks: ranks, all_reduce_sum=lambda t, h: None)


def test_registry_creates_each_group_once_in_sorted_order():
    frag = P.plan_canonical_fragments(_all_descs(), [0, 1])
    seen = []
    reg = B.ProcessGroupRegistry(frag.process_groups, lambda ranks: seen.append(ranks) or ranks)
    reg.initialize()
    reg.initialize()
    assert seen == sorted(seen) and reg.creation_count == len(seen) == reg.group_count
    with pytest.raises(KeyError):
        reg.handle("pg-unknown")
