"""Sharding-spec algebra: which collective connects two placements, duals, and execution on Gloo."""
import pytest
import torch

from eth_b200.parallel.resharding import ReshardStep, plan_reshard, reshard_bytes
from eth_b200.search.model_ops import full_op_list, get_op_spec
from tests.helpers.multiproc import run_ranks


def test_op_specs_chain_without_communication_for_algo0():
    tp, dp = 4, 2
    ops = full_op_list(1)
    for a, b in zip(ops, ops[1:]):
        out, inp = get_op_spec(a, tp, dp, 0, False), get_op_spec(b, tp, dp, 0, True)
        step = plan_reshard(out, inp)
        # column -> row pairs need nothing in between; row outputs are reduced inside the op
        assert step.primitive in ("identity", "split"), (a, b, step)
    assert len(full_op_list(3)) == 33 and len(full_op_list(3, legacy=True)) == 42


@pytest.mark.parametrize("src,dst,prim", [
    ({"R": 4, "V": 1, "dims": [1, 1, 1]}, {"R": 1, "V": 1, "dims": [1, 1, 4]}, "split"),
    ({"R": 1, "V": 4, "dims": [1, 1, 1]}, {"R": 4, "V": 1, "dims": [1, 1, 1]}, "all_reduce"),
    ({"R": 1, "V": 4, "dims": [1, 1, 1]}, {"R": 1, "V": 1, "dims": [1, 4, 1]}, "reduce_scatter"),
    ({"R": 1, "V": 1, "dims": [1, 1, 4]}, {"R": 4, "V": 1, "dims": [1, 1, 1]}, "all_gather"),
    ({"R": 1, "V": 1, "dims": [1, 1, 4]}, {"R": 1, "V": 1, "dims": [4, 1, 1]}, "all_to_all"),
])
def test_primitive_choice_and_dual(src, dst, prim):
    step = plan_reshard(src, dst)
    assert step.primitive == prim and step.group_size == 4
    if prim in ("split", "all_gather", "all_to_all"):      # nothing turns back into partial sums
        assert plan_reshard(dst, src).primitive == step.dual().primitive
    assert reshard_bytes(step, 1000.0) == (0.0 if prim == "split" else (1500.0 if prim == "all_reduce" else 750.0))


def test_mismatched_sizes_are_rejected():
    with pytest.raises(ValueError):
        plan_reshard({"R": 2, "V": 1, "dims": [1, 1, 1]}, {"R": 1, "V": 1, "dims": [1, 1, 4]})


def _run_prims(rank, world):
    from eth_b200.parallel.resharding import apply_reshard
    full = torch.arange(4 * 6 * 8, dtype=torch.float32).view(4, 6, 8)
    out = {}
    shard = full.chunk(world, dim=2)[rank].contiguous()
    out["all_gather"] = torch.equal(apply_reshard(shard, ReshardStep("all_gather", world, src_dim=2)), full)
    out["split"] = torch.equal(apply_reshard(full, ReshardStep("split", world, dst_dim=1)), full.chunk(world, 1)[rank])
    out["all_reduce"] = torch.equal(apply_reshard(full, ReshardStep("all_reduce", world)), full * world)
    out["reduce_scatter"] = torch.equal(apply_reshard(full, ReshardStep("reduce_scatter", world, dst_dim=0)),
                                        (full * world).chunk(world, 0)[rank])
    a2a = apply_reshard(shard, ReshardStep("all_to_all", world, src_dim=2, dst_dim=0))
    out["all_to_all"] = torch.equal(a2a, full.chunk(world, 0)[rank])
    return out


def test_primitives_on_gloo():
    for res in run_ranks(2, _run_prims):
        assert all(res.values()), res


def _autograd_adapters(rank, world):
    """Column- then row-parallel MLP written with the autograd adapters, against the same MLP on
    one rank; and a split / gather round trip whose backward runs the duals."""
    import torch
    from eth_b200.parallel import resharding as R
    torch.manual_seed(0)
    x = torch.randn(6, 8, dtype=torch.float64)
    w1, w2 = torch.randn(16, 8, dtype=torch.float64), torch.randn(8, 16, dtype=torch.float64)
    g = torch.randn(6, 8, dtype=torch.float64)
    # one-rank oracle
    xo, w1o, w2o = (t.clone().requires_grad_(True) for t in (x, w1, w2))
    (torch.tanh(xo @ w1o.t()) @ w2o.t()).backward(g)
    # two ranks: W1 cut along its rows, W2 along its columns
    xr = x.clone().requires_grad_(True)
    w1r = w1.chunk(world, 0)[rank].clone().requires_grad_(True)
    w2r = w2.chunk(world, 1)[rank].clone().requires_grad_(True)
    y = R.reduce_from_region(torch.tanh(R.copy_to_region(xr) @ w1r.t()) @ w2r.t())
    y.backward(g)
    errs = [float((xr.grad - xo.grad).abs().max()), float((w1r.grad - w1o.grad.chunk(world, 0)[rank]).abs().max()),
            float((w2r.grad - w2o.grad.chunk(world, 1)[rank]).abs().max())]
    # placement algebra end to end: replicated -> hidden split -> replicated, gradients flow through the duals
    rep, split = {"R": world, "V": 1, "dims": [1, 1, 1]}, {"R": 1, "V": 1, "dims": [1, 1, world]}
    t = torch.randn(2, 3, 4 * world, dtype=torch.float64, generator=torch.Generator().manual_seed(5)).requires_grad_(True)
    back = R.tensor_adapter(R.tensor_adapter(t, rep, split) * (rank + 1.0), split, rep)
    back.sum().backward()
    expect = torch.cat([t.detach().chunk(world, 2)[r] * (r + 1.0) for r in range(world)], 2)
    errs.append(float((back.detach() - expect).abs().max()))
    # backward: the gather's dual keeps this rank's slice of the (replicated) gradient, the scale is
    # applied, and the split's dual gathers every rank's slice gradient into the full tensor
    want = torch.cat([torch.full_like(c, r + 1.0) for r, c in enumerate(t.detach().chunk(world, 2))], 2)
    errs.append(float((t.grad - want).abs().max()))
    return errs


def test_autograd_adapters_on_gloo():
    for errs in run_ranks(2, _autograd_adapters):
        assert max(errs) < 1e-12, errs
