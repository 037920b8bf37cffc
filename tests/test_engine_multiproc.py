"""Topology independence: after N optimizer steps every parallel layout holds the same logical
parameters as a single-rank run over the same global batch (the evidence protocol of the
reference, tools/validation/compare_numerical_evidence.py, run here on CPU ranks over Gloo)."""
import pytest
import torch

from eth_b200.contract.config import make_config, make_pipe, manifest_size
from tests.helpers.multiproc import run_ranks

LAYERS, HIDDEN, HEADS, SEQ, VOCAB = 2, 32, 4, 16, 96
N_OPS = manifest_size(LAYERS)


def _config(pipes):
    return make_config(pipes, num_layers=LAYERS, hidden_size=HIDDEN, num_attention_heads=HEADS, seq_length=SEQ)


def _train(rank, world, config, steps, mode):
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    argv = ["--hidden-dropout", "0.0", "--device", "cpu", "--vocab-size", str(VOCAB),
            "--make-vocab-size-divisible-by", "8", "--lr", "1e-2", "--lr-warmup-fraction", "0.0",
            "--lr-decay-style", "constant", "--grad-sync-mode", mode, "--grad-sync-bucket-size-mb", "1",
            "--distributed-backend", "gloo"]
    args = parse_args(argv, config=config, rank=rank, world_size=world)
    # identical vocabulary padding in every layout so logical shapes agree
    eng = TrainEngine(args, device="cpu")
    losses, norms = [], []
    for _ in range(steps):
        st = eng.train_step()
        losses.append(eng.reduced_loss())
        norms.append(st["grad_norm"])
    shards = []
    for e in eng.stage.unique_entries():
        shards.append((e.spec.logical_id, e.spec.full_shape, e.spec.partition_dim, eng.pstate.tp_size,
                       eng.pstate.tp_rank, eng.pstate.pipeline_id, eng.pstate.dp_rank, e.param.detach().clone()))
    return {"losses": losses, "norms": norms, "shards": shards,
            "collectives": eng.grad_sync.executor.collectives_issued}


def _logical(results, pipeline=0, dp=0):
    """Reassemble full logical tensors from one (pipeline, dp) replica."""
    parts = {}
    for res in results:
        for lid, full, pdim, tp, tpr, pid, dpr, t in res["shards"]:
            if pid == pipeline and dpr == dp:
                parts.setdefault(lid, {})[tpr] = (pdim, tp, t)
    out = {}
    for lid, by in parts.items():
        pdim, tp, _ = next(iter(by.values()))
        if pdim < 0 or tp == 1:
            out[lid] = by[min(by)][2]
        else:
            out[lid] = torch.cat([by[r][2] for r in range(tp)], pdim)
    return out


LAYOUTS = {
    "tp2": (2, [make_pipe([N_OPS], [2], [1], gbs=8, mbs=4)]),
    "dp2": (2, [make_pipe([N_OPS], [1], [2], gbs=8, mbs=4)]),
    "dp4": (4, [make_pipe([N_OPS], [1], [4], gbs=8, mbs=4)]),
    "pp2": (2, [make_pipe([11, N_OPS - 11], [1, 1], [1, 1], gbs=8, mbs=4)]),
    "pp2-midlayer-cut": (2, [make_pipe([6, N_OPS - 6], [1, 1], [1, 1], gbs=8, mbs=4)]),
    "pp2-tp2-to-dp2": (4, [make_pipe([11, N_OPS - 11], [2, 1], [1, 2], gbs=8, mbs=4)]),
    "two-pipelines-hetero": (3, [make_pipe([N_OPS], [2], [1], gbs=4, mbs=4), make_pipe([N_OPS], [1], [1], gbs=4, mbs=2)]),
    "pp3-1f1b": (3, [make_pipe([11, 10, N_OPS - 21], [1, 1, 1], [1, 1, 1], gbs=8, mbs=2)]),
    # algo 1: the four tensor-parallel GEMMs of a stage use the swapped sharding (qkv / GEMM-1 row-parallel,
    # dense / GEMM-2 column-parallel) and convert placements at their own inputs and outputs
    "tp2-algo1": (2, [dict(make_pipe([N_OPS], [2], [1], gbs=8, mbs=4, algo=[1]), resharding_stages=[True])]),
    "pp2-tp2-algo1-then-algo0": (4, [dict(make_pipe([7, N_OPS - 7], [2, 2], [1, 1], gbs=8, mbs=4, algo=[1, 0]),
                                          resharding_stages=[True, False])]),
}


@pytest.fixture(scope="module")
def oracle():
    cfg = _config([make_pipe([N_OPS], [1], [1], gbs=8, mbs=4)])
    return run_ranks(1, _train, cfg, 2, "block")


@pytest.mark.parametrize("name", sorted(LAYOUTS))
def test_layout_matches_single_rank(name, oracle):
    world, pipes = LAYOUTS[name]
    results = run_ranks(world, _train, _config(pipes), 2, "block")
    ref = _logical(oracle)
    merged = {}
    for res in results:
        for lid, full, pdim, tp, tpr, pid, dpr, t in res["shards"]:
            merged.setdefault((lid, pid, dpr), {})[tpr] = (pdim, tp, t)
    for (lid, pid, dpr), by in merged.items():
        pdim, tp, _ = next(iter(by.values()))
        full = by[min(by)][2] if (pdim < 0 or tp == 1) else torch.cat([by[r][2] for r in range(tp)], pdim)
        err = (full - ref[lid]).norm() / (ref[lid].norm() + 1e-12)
        assert err < 2e-4, (name, lid, pid, dpr, float(err))
    for a, b in zip(results[-1]["losses"], oracle[0]["losses"]):
        assert abs(a - b) < 1e-4
    for a, b in zip(results[0]["norms"], oracle[0]["norms"]):
        assert abs(a - b) / b < 1e-3


def test_block_mode_issues_fewer_collectives_than_tensor_mode():
    world, pipes = LAYOUTS["dp2"]
    block = run_ranks(world, _train, _config(pipes), 1, "block")
    tensor = run_ranks(world, _train, _config(pipes), 1, "tensor")
    assert block[0]["collectives"] < tensor[0]["collectives"]
    for (a, b) in zip(block[0]["shards"], tensor[0]["shards"]):
        assert torch.allclose(a[-1], b[-1], atol=1e-6)


# ------------------------------------------------------------------ interleaved 1F1B
def _train_interleaved(rank, world, config, steps, factor):
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    argv = ["--hidden-dropout", "0.0", "--device", "cpu", "--vocab-size", str(VOCAB),
            "--make-vocab-size-divisible-by", "8", "--lr", "1e-2", "--lr-warmup-fraction", "0.0",
            "--lr-decay-style", "constant", "--grad-sync-mode", "block", "--grad-sync-bucket-size-mb", "1",
            "--distributed-backend", "gloo", "--interleave-factor", str(factor)]
    args = parse_args(argv, config=config, rank=rank, world_size=world)
    eng = TrainEngine(args, device="cpu")
    losses, norms = [], []
    for _ in range(steps):
        st = eng.train_step()
        losses.append(eng.reduced_loss())
        norms.append(st["grad_norm"])
    params = {lid: p.detach().clone() for lid, p in eng.stage.named_parameters()}
    return {"losses": losses, "norms": norms, "params": params, "chunks": eng.stage.chunk_ranges}


@pytest.mark.parametrize("name,world,stage_ops,factor,gbs,mbs", [
    ("pp2-v2", 2, [11, N_OPS - 11], 2, 8, 2),           # 4 micro-batches, chunks cut inside the layers
    ("pp2-v2-all-warmup", 2, [11, N_OPS - 11], 2, 4, 2),  # micro-batches == stages: no steady phase
    ("pp3-v2", 3, [7, 7, N_OPS - 14], 2, 12, 2),        # 6 micro-batches, uneven op-granular chunks
])
def test_interleaved_schedule_matches_single_rank(name, world, stage_ops, factor, gbs, mbs):
    single = run_ranks(1, _train_interleaved, _config([make_pipe([N_OPS], [1], [1], gbs=gbs, mbs=mbs)]), 2, 1)[0]
    pipe = make_pipe(stage_ops, [1] * world, [1] * world, gbs=gbs, mbs=mbs)
    results = run_ranks(world, _train_interleaved, _config([pipe]), 2, factor)
    # every rank holds `factor` chunks and together they cover the model exactly once, in virtual-stage order
    ranges = sorted(r for res in results for r in res["chunks"])
    assert all(len(res["chunks"]) == factor for res in results)
    assert ranges[0][0] == 0 and ranges[-1][1] == N_OPS and all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    virtual = [results[s]["chunks"][c] for c in range(factor) for s in range(world)]
    assert virtual == ranges
    merged = {}
    for res in results:
        merged.update(res["params"])
    for lid, ref in single["params"].items():
        err = (merged[lid] - ref).norm() / (ref.norm() + 1e-12)
        assert err < 2e-4, (name, lid, float(err))
    for a, b in zip(results[-1]["losses"], single["losses"]):
        assert abs(a - b) < 1e-4
    for a, b in zip(results[0]["norms"], single["norms"]):
        assert abs(a - b) / b < 1e-3


def _tp_feed(rank, world, prefix):
    """TP2 engine on an indexed dataset: rank 0 of the group reads, rank 1 receives the broadcast."""
    from types import SimpleNamespace
    from eth_b200.data.provider import providers_from_args
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    config = _config([make_pipe([N_OPS], [2], [1], gbs=4, mbs=2)])
    argv = ["--hidden-dropout", "0.0", "--device", "cpu", "--vocab-size", str(VOCAB), "--make-vocab-size-divisible-by",
            "8", "--distributed-backend", "gloo", "--data-path", prefix, "--split", "1,0,0", "--train-iters", "2"]
    args = parse_args(argv, config=config, rank=rank, world_size=world)
    eng = TrainEngine(args, device="cpu")
    eng.data_provider, eng.eval_data_provider = providers_from_args(args, eng.pstate, None)
    tokens, labels, mask = eng.get_batch(1)
    eng.train_step()
    reads_data = getattr(eng.data_provider, "inner", None) is not None
    return {"tokens": tokens.clone(), "labels": labels.clone(), "mask": mask.clone(), "reads": reads_data,
            "loss": eng.reduced_loss()}


def test_dataset_batches_are_broadcast_inside_a_tp_group(tmp_path):
    import numpy as np
    from eth_b200.data.indexed_dataset import MMapIndexedDatasetBuilder
    prefix = str(tmp_path / "toy")
    rng = np.random.RandomState(0)
    b = MMapIndexedDatasetBuilder(prefix + ".bin", dtype=np.uint16)
    for _ in range(60):
        b.add_item(rng.randint(1, VOCAB, size=rng.randint(5, 30)))
        b.end_document()
    b.finalize(prefix + ".idx")
    r0, r1 = run_ranks(2, _tp_feed, prefix)
    assert r0["reads"] and not r1["reads"]
    for key in ("tokens", "labels", "mask"):
        assert torch.equal(r0[key], r1[key])
    assert torch.equal(r0["tokens"][:, 1:], r0["labels"][:, :-1])
    assert r0["loss"] == r1["loss"] and r0["loss"] == r0["loss"]


def test_algo1_needs_a_resharding_stage():
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    cfg = _config([make_pipe([N_OPS], [2], [1], gbs=8, mbs=4, algo=[1])])
    args = parse_args(["--device", "cpu", "--vocab-size", str(VOCAB), "--distributed-backend", "gloo"], config=cfg,
                      rank=0, world_size=2)
    with pytest.raises(ValueError, match="resharding_stages"):
        TrainEngine(args, device="cpu")
