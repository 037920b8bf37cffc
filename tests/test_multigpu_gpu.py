"""Multi-GPU kernels and engine paths (NCCL ranks on 2+ GPUs of one node; skipped with fewer)."""
import pytest
import torch

from tests.helpers.multiproc import run_ranks

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    """max(norm-wise relative error, largest element error over the largest reference magnitude)."""
    a, b = a.float(), b.float()
    err = max(((a - b).norm() / (b.norm() + 1e-12)).item(), ((a - b).abs().max() / (b.abs().max() + 1e-12)).item())
    return err if err == err else float("inf")   # a NaN anywhere must fail every `< tolerance` check


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _fused_gemm_ar(rank, world, shapes, poison=False):
    import os
    import torch.distributed as dist
    if poison:   # staging areas start as NaN patterns: a slot read before it was written shows up
        os.environ["ETHB_POISON_STAGING"] = "1"
    from eth_b200.ops import native
    from eth_b200.parallel.fused_tp import FusedTPBackend
    dev = torch.device("cuda", rank)
    be = FusedTPBackend(tuple(range(world)), rank, None, dev, max_tokens=4096, hidden=2048, dtype=torch.bfloat16)
    errs = []
    for (m, n, k, b_mn, reps) in shapes:
        for rep in range(reps):
            g = torch.Generator(device=dev).manual_seed(1000 * rank + rep)
            a = torch.randn(m, k, device=dev, dtype=torch.bfloat16, generator=g)
            w = torch.randn((k, n) if b_mn else (n, k), device=dev, dtype=torch.bfloat16, generator=g) * 0.05
            out = be.gemm_all_reduce(a, w, b_mn=b_mn).clone()
            ref = a.float() @ (w.float() if b_mn else w.float().t())
            dist.all_reduce(ref)
            errs.append(_rel_err(out, ref))
    native.check_status()
    # every rank must hold the same bits
    chk = out.float().sum().reshape(1).clone()
    lst = [torch.zeros_like(chk) for _ in range(world)]
    dist.all_gather(lst, chk)
    same = all(torch.equal(lst[0], x) for x in lst)
    be.close()
    return {"errs": errs, "same": same}


def test_fused_gemm_allreduce_two_gpus():
    _need(2)
    shapes = [(256, 512, 256, False, 2), (4096, 2048, 1024, False, 3), (1000, 2048, 512, True, 2), (4096, 2048, 4096, True, 2)]
    for poison in (False, True):
        res = run_ranks(2, _fused_gemm_ar, shapes, poison, backend="nccl")
        for r in res:
            assert all(e < 1e-2 for e in r["errs"]), (poison, r["errs"])   # a NaN error compares false
            assert r["same"]


def _peer_allreduce(rank, world):
    import torch.distributed as dist
    from eth_b200.ops import native
    from eth_b200.parallel.peer_memory import SymmetricBuffer
    dev = torch.device("cuda", rank)
    n = 1_000_003
    buf = SymmetricBuffer(n * 4, tuple(range(world)), rank, None, dev)
    flags = SymmetricBuffer(64 * 4, tuple(range(world)), rank, None, dev)
    mine = buf.tensor((n,), torch.float32)
    out = torch.empty(n, device=dev)
    acc = torch.zeros(2, device=dev)
    errs = []
    for epoch in (1, 2, 3):
        src = torch.randn(n, device=dev) * (rank + 1)
        mine.copy_(src)
        ref = src.clone()
        dist.all_reduce(ref)
        ref *= 0.5
        acc.zero_()
        native.lib().peer_allreduce(buf.ptrs, flags.ptrs, rank, epoch, n, 0, 0.5, out, acc, 1.0, native.status(dev))
        errs.append(_rel_err(out, ref))
        errs.append(abs(acc[0].item() - ref.pow(2).sum().item()) / ref.pow(2).sum().item())
    native.check_status()
    return errs


def test_peer_allreduce_two_gpus():
    _need(2)
    for errs in run_ranks(2, _peer_allreduce, backend="nccl"):
        assert all(e < 1e-4 for e in errs), errs


def _engine_loss(rank, world, tp, algo=0):
    from eth_b200.contract.config import make_config, make_pipe, manifest_size
    from eth_b200.ops import native
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    layers = 2
    pipe = make_pipe([manifest_size(layers)], [tp], [world // tp], gbs=8, mbs=4, algo=[algo])
    pipe["resharding_stages"] = [bool(algo)]
    cfg = make_config([pipe], num_layers=layers, hidden_size=512, num_attention_heads=4, seq_length=256)
    args = parse_args(["--bf16", "--hidden-dropout", "0.0", "--vocab-size", "2000", "--lr", "1e-3",
                       "--lr-warmup-fraction", "0.0", "--make-vocab-size-divisible-by", "64"],
                      config=cfg, rank=rank, world_size=world)
    eng = TrainEngine(args)
    out = []
    for _ in range(3):
        st = eng.train_step()
        out.append((eng.reduced_loss(), st["grad_norm"]))
    native.check_status()
    return out


def test_engine_tp2_and_dp2_match_single_gpu():
    _need(2)
    single = run_ranks(1, _engine_loss, 1, backend="nccl")[0]
    tp2 = run_ranks(2, _engine_loss, 2, backend="nccl")[0]
    dp2 = run_ranks(2, _engine_loss, 1, backend="nccl")[0]
    swapped = run_ranks(2, _engine_loss, 2, 1, backend="nccl")[0]   # TP2 with the GEMMs in their other sharding
    for (l1, n1), (l2, n2), (l3, n3), (l4, n4) in zip(single, tp2, dp2, swapped):
        assert abs(l1 - l2) < 3e-2 and abs(l1 - l3) < 3e-2 and abs(l1 - l4) < 3e-2, (single, tp2, dp2, swapped)
        assert max(abs(n1 - n2), abs(n1 - n3), abs(n1 - n4)) / n1 < 5e-2, (single, tp2, dp2, swapped)


def _fused_rs_ag(rank, world):
    import torch.distributed as dist
    from eth_b200.ops import native
    from eth_b200.parallel.fused_tp import FusedTPBackend
    dev = torch.device("cuda", rank)
    dt = torch.bfloat16
    be = FusedTPBackend(tuple(range(world)), rank, None, dev, max_tokens=4096, hidden=2048, dtype=dt)
    out = {"rs": [], "ag": []}
    # GEMM + reduce-scatter: rows [rank * M / W, ...) of the summed product, with bias and a sharded residual
    for (m, n, k, b_mn) in [(512, 512, 256, False), (4096, 2048, 1024, False), (2048, 2048, 3072, True)]:
        for rep in range(2):
            g = torch.Generator(device=dev).manual_seed(77 * rank + rep)
            a = torch.randn(m, k, device=dev, dtype=dt, generator=g)
            w = torch.randn((k, n) if b_mn else (n, k), device=dev, dtype=dt, generator=g) * 0.05
            bias = torch.randn(n, device=dev, dtype=dt, generator=torch.Generator(device=dev).manual_seed(5))
            res = torch.randn(m // world, n, device=dev, dtype=dt, generator=g)
            got = be.gemm_reduce_scatter(a, w, b_mn=b_mn, bias=bias, residual=res).clone()
            ref = a.float() @ (w.float() if b_mn else w.float().t())
            dist.all_reduce(ref)
            rows = m // world
            ref = ref[rank * rows:(rank + 1) * rows] + bias.float() + res.float()
            out["rs"].append(_rel_err(got, ref))
    # all-gather + GEMM: every rank contributes a row block of the operand
    for (m, n, k, b_mn) in [(512, 768, 256, False), (4096, 3072, 2048, False), (2048, 1024, 2048, True)]:
        for rep in range(2):
            g = torch.Generator(device=dev).manual_seed(31 * rank + rep)
            full, mine = be.gather_buffer(m, k)
            block = torch.randn(m // world, k, device=dev, dtype=dt, generator=g)
            mine.copy_(block)
            w = torch.randn((k, n) if b_mn else (n, k), device=dev, dtype=dt, generator=torch.Generator(device=dev).manual_seed(9)) * 0.05
            bias = torch.randn(n, device=dev, dtype=dt, generator=torch.Generator(device=dev).manual_seed(6))
            got = be.gemm_all_gather(full, w, b_mn=b_mn, bias=bias)
            blocks = [torch.empty_like(block) for _ in range(world)]
            dist.all_gather(blocks, block)
            a_ref = torch.cat(blocks).float()
            ref = a_ref @ (w.float() if b_mn else w.float().t()) + bias.float()
            out["ag"].append(_rel_err(got, ref))
            out["ag"].append(float(not torch.equal(full, torch.cat(blocks))))   # gathered operand itself
    native.check_status()
    be.close()
    return out


def test_fused_reduce_scatter_and_all_gather_gemm_two_gpus():
    _need(2)
    res = run_ranks(2, _fused_rs_ag, backend="nccl")
    for r in res:
        assert all(e < 1e-2 for e in r["rs"]), r["rs"]
        assert all(e < 1e-2 for e in r["ag"]), r["ag"]


def _peer_reduce_pieces(rank, world):
    """Two-shot in-place reduction of pieces (whole runs and a strided 2-D slice) of a symmetric buffer."""
    import torch.distributed as dist
    from eth_b200.ops import native
    from eth_b200.parallel.peer_memory import SymmetricBuffer
    dev = torch.device("cuda", rank)
    out = {}
    for dt, code, tol in ((torch.float32, 0, 1e-6), (torch.float16, 1, 2e-3), (torch.bfloat16, 2, 1.6e-2)):
        n = 1 << 20
        esz = torch.empty((), dtype=dt).element_size()
        buf = SymmetricBuffer(n * esz, tuple(range(world)), rank, None, dev)
        flags = SymmetricBuffer(64 * 4, tuple(range(world)), rank, None, dev)
        mine = buf.tensor((n,), dt)
        # pieces: a long run, a short run, and 96 rows of 64 elements with row stride 256
        pieces = [(0, 1, 300_000, 300_000), (400_000, 1, 4096, 4096), (500_000, 96, 64, 256)]
        table = torch.tensor(pieces, dtype=torch.int64, device=dev)
        errs = []
        for epoch in (1, 2):
            src = (torch.randn(n, device=dev) * (rank + 1)).to(dt)
            mine.copy_(src)
            ref = src.float().clone()
            dist.all_reduce(ref)
            ref *= 0.5
            dist.barrier()
            st = native.status(dev)
            native.lib().peer_flags(flags.ptrs, rank, epoch, 0, 0, st)
            native.lib().peer_reduce_pieces(buf.ptrs, flags.ptrs, rank, epoch, table, code, 0.5)
            native.lib().peer_flags(flags.ptrs, rank, epoch, -1, 8, st)
            got = mine.float()
            touched = torch.zeros(n, dtype=torch.bool, device=dev)
            for off, rows, run, stride in pieces:
                for r in range(rows):
                    touched[off + r * stride: off + r * stride + run] = True
            errs.append(float((got[touched] - ref[touched]).abs().max() / ref[touched].abs().max()))
            errs.append(float((got[~touched] - src.float()[~touched]).abs().max()))   # untouched elements intact
            torch.cuda.synchronize()
            dist.barrier()
        native.check_status()
        out[str(dt)] = (errs, tol)
        buf.close()
        flags.close()
    return out


def test_peer_reduce_pieces_two_gpus():
    _need(2)
    for res in run_ranks(2, _peer_reduce_pieces, backend="nccl"):
        for name, (errs, tol) in res.items():
            assert errs[0] <= tol and errs[2] <= tol, (name, errs)
            assert errs[1] == 0.0 and errs[3] == 0.0, (name, errs)


def _engine_dp2_params(rank, world, extra):
    from eth_b200.contract.config import make_config, make_pipe, manifest_size
    from eth_b200.ops import native
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    layers = 2
    cfg = make_config([make_pipe([manifest_size(layers)], [1], [world], gbs=16, mbs=8)], num_layers=layers,
                      hidden_size=512, num_attention_heads=4, seq_length=256)
    args = parse_args(["--bf16", "--hidden-dropout", "0.1", "--vocab-size", "2000", "--lr", "1e-3",
                       "--lr-warmup-fraction", "0.0", "--make-vocab-size-divisible-by", "64",
                       "--grad-sync-bucket-size-mb", "1"] + list(extra), config=cfg, rank=rank, world_size=world)
    eng = TrainEngine(args)
    direct = sum(1 for b in eng.grad_sync.executor.buckets
                 if eng.grad_sync.executor.uses_peer_backend(b) and eng.grad_sync.executor._peer.is_direct(b))
    for _ in range(3):
        eng.train_step()
    native.check_status()
    flat = eng.stage.param_buf.detach().float().clone()
    return {"params": flat.cpu(), "direct": direct, "overlapped": len(eng._overlap_by_op), "loss": eng.reduced_loss()}


def test_engine_dp2_overlapped_peer_reduction_matches_nccl():
    """Gradient buckets reduced in place by the peer kernel while backward still runs (the default,
    with weight gradients on their side stream) give the parameters of the plain NCCL path."""
    _need(2)
    over = run_ranks(2, _engine_dp2_params, (), backend="nccl")
    plain = run_ranks(2, _engine_dp2_params, ("--no-overlap-grad-sync",), backend="nccl")
    nccl = run_ranks(2, _engine_dp2_params, ("--grad-sync-backend", "collective"), backend="nccl")
    assert over[0]["direct"] > 0 and over[0]["overlapped"] > 0 and plain[0]["overlapped"] == 0
    assert torch.equal(over[0]["params"], over[1]["params"])            # replicas stay identical
    for a in (over, plain):
        diff = (a[0]["params"] - nccl[0]["params"]).abs()
        # bf16 weights: a different summation order may flip the last bit of a few values (1 ulp at 1.0 = 2^-7)
        assert diff.max().item() <= 2 ** -7 and diff.mean().item() < 1e-5, (diff.max().item(), diff.mean().item())
        assert abs(a[0]["loss"] - nccl[0]["loss"]) < 2e-2


def _engine_pp2(rank, world, backend, cut):
    from eth_b200.contract.config import make_config, make_pipe, manifest_size
    from eth_b200.ops import native
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    layers = 2
    n = manifest_size(layers)
    cfg = make_config([make_pipe([cut, n - cut], [1, 1], [1, 1], gbs=12, mbs=2)], num_layers=layers,
                      hidden_size=512, num_attention_heads=4, seq_length=256)
    args = parse_args(["--bf16", "--hidden-dropout", "0.1", "--vocab-size", "2000", "--lr", "1e-3",
                       "--lr-warmup-fraction", "0.0", "--make-vocab-size-divisible-by", "64", "--no-async-wgrad",
                       "--p2p-backend", backend], config=cfg, rank=rank, world_size=world)
    eng = TrainEngine(args)
    losses = []
    for _ in range(3):
        eng.train_step()
        losses.append(eng.reduced_loss())
    eng.eval_step()                     # forward-only passes stay on the NCCL channels
    eval_loss = eng.reduced_loss()
    eng.train_step()                    # and training continues on the ring afterwards
    losses.append(eng.reduced_loss())
    torch.cuda.synchronize()
    native.check_status()
    return {"backend": eng.p2p_backend, "losses": losses, "eval": eval_loss,
            "params": eng.stage.param_buf.detach().float().cpu().clone()}


@pytest.mark.parametrize("cut", [11, 6])     # a layer boundary; inside a layer (hidden + bias vector + residual)
def test_pipeline_transfers_through_peer_memory_match_nccl(cut):
    """PP2 with six micro-batches (more than the ring has slots): activations and gradients that
    travel as copy-engine copies into the neighbour's ring slots, awaited through flags, train like
    the NCCL isend / irecv path."""
    _need(2)
    peer = run_ranks(2, _engine_pp2, "peer", cut, backend="nccl")
    nccl = run_ranks(2, _engine_pp2, "nccl", cut, backend="nccl")
    assert peer[0]["backend"] == "peer" and nccl[0]["backend"] == "nccl"
    for r in (0, 1):
        diff = (peer[r]["params"] - nccl[r]["params"]).abs()
        # same kernels on the same data: only the embedding's atomic accumulation order may differ
        assert diff.max().item() <= 2 ** -7 and diff.mean().item() < 1e-5, (r, diff.max().item(), diff.mean().item())
    for a, b in zip(peer[1]["losses"] + [peer[1]["eval"]], nccl[1]["losses"] + [nccl[1]["eval"]]):
        assert abs(a - b) < 2e-3 and a == a, (peer[1], nccl[1])
