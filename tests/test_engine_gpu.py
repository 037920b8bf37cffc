"""Engine-level GPU checks of the stream-parallel execution options."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(extra):
    from eth_b200.contract.config import uniform_config
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    model = dict(model_size="tiny", num_layers=3, hidden_size=256, num_attention_heads=4, seq_length=256,
                 max_position_embeddings=256)
    config = uniform_config(model, pp=1, tp=1, dp=1, gbs=10, mbs=2)
    args = parse_args(["--bf16", "--vocab-size", "1024", "--train-iters", "3", "--hidden-dropout", "0.1"] + extra,
                      config=config, rank=0, world_size=1, local_rank=0)
    return TrainEngine(args, device=torch.device("cuda", 0))


def _run(extra):
    from eth_b200.ops import native
    eng = _engine(extra)
    losses = []
    for _ in range(3):
        eng.train_step()
        losses.append(eng.reduced_loss())
    torch.cuda.synchronize()
    native.check_status()
    return eng.stage.param_buf.float().clone(), losses


def test_async_wgrad_matches_single_stream():
    """Weight gradients on a side stream keep the accumulation order per weight, so training must
    follow the single-stream run: same first loss, and parameters that differ no more than two
    single-stream runs differ from each other (the embedding gradient uses floating-point atomics)."""
    p0, l0 = _run(["--no-async-wgrad"])
    p1, l1 = _run(["--no-async-wgrad"])
    p2, l2 = _run([])
    assert l0[0] == l1[0] == l2[0]
    noise = (p0 - p1).abs().max().item()
    diff = (p0 - p2).abs().max().item()
    assert diff <= max(4 * noise, 2e-3), (noise, diff, l0, l2)
    assert all(abs(a - b) <= max(1e-3, 4 * abs(a - c)) for a, b, c in zip(l0, l2, l1)), (l0, l1, l2)


def test_deferred_column_sums_train_like_per_micro_batch_sums():
    """Summing LayerNorm-weight and bias gradients once per step (partial sums kept in per-op slabs
    over the five micro-batches) trains like summing them after every micro-batch."""
    p0, l0 = _run(["--no-async-wgrad", "--no-deferred-colsums"])
    p1, l1 = _run(["--no-async-wgrad", "--no-deferred-colsums"])
    p2, l2 = _run(["--no-async-wgrad"])
    assert l0[0] == l2[0]
    noise = (p0 - p1).abs().max().item()
    diff = (p0 - p2).abs().max().item()
    assert diff <= max(4 * noise, 2e-3), (noise, diff, l0, l2)
    assert all(abs(a - b) <= max(1e-3, 4 * abs(a - c)) for a, b, c in zip(l0, l2, l1)), (l0, l1, l2)


@pytest.mark.parametrize("dtype_flag,tol", [("--bf16", 4e-2), ("--fp16", 1.5e-2)])
def test_native_stage_program_matches_fp32_oracle(dtype_flag, tol):
    """Forward + backward of the sm_100a stage program (tcgen05 GEMMs with fused epilogues, flash
    attention, LayerNorm, cross entropy, embedding) against a plain fp32 autograd GPT on the CPU that
    starts from the same 16-bit weights: loss, every parameter gradient, and one AdamW step."""
    from eth_b200.contract.config import make_config, make_pipe, manifest_size
    from eth_b200.ops import native
    from eth_b200.runtime import schedules
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    from tests.helpers.oracle_gpt import oracle_loss
    layers = 2
    cfg = make_config([make_pipe([manifest_size(layers)], [1], [1], gbs=4, mbs=2)], num_layers=layers,
                      hidden_size=256, num_attention_heads=4, seq_length=128)
    argv = [dtype_flag, "--hidden-dropout", "0.0", "--vocab-size", "1000", "--make-vocab-size-divisible-by", "8",
            "--clip-grad", "1.0", "--lr", "1e-3", "--lr-warmup-fraction", "0.0", "--lr-decay-style", "constant",
            "--no-async-wgrad"]
    if dtype_flag == "--fp16":
        argv += ["--loss-scale", "256"]
    args = parse_args(argv, config=cfg, rank=0, world_size=1, local_rank=0)
    eng = TrainEngine(args, device=torch.device("cuda", 0))
    mcfg = eng.model_cfg
    params = {lid: p.detach().float().cpu().clone().requires_grad_(True) for lid, p in eng.stage.named_parameters()}
    total = 0.0
    for i in range(eng.pstate.num_microbatches):
        tokens, labels, mask = (t.cpu() for t in eng.get_batch(i))
        loss, _ = oracle_loss(params, tokens, labels, mask, mcfg, args.nominal_global_loss_scale)
        total = total + loss
    total.backward()
    eng.optimizer.zero_grad()
    eng.loss_acc.zero_()
    schedules.forward_backward_no_pipelining(eng, eng.pstate.num_microbatches)
    torch.cuda.synchronize()
    native.check_status()
    scale = eng.scaler.value() if eng.scaler is not None else 1.0
    got_loss = float(eng.loss_acc[0]) / args.nominal_global_loss_scale
    assert abs(got_loss - float(total)) < 2e-2 * abs(float(total)), (got_loss, float(total))
    for lid, p in eng.stage.named_parameters():
        ref = params[lid].grad
        got = p.main_grad.float().cpu() / scale
        err = (got - ref).norm() / (ref.norm() + 1e-12)
        worst = (got - ref).abs().max() / (ref.abs().max() + 1e-12)
        assert err < tol and worst < 4 * tol, (lid, float(err), float(worst))
    # one optimizer step against torch AdamW on the oracle gradients (same clip, same decay groups)
    decay = [v for k, v in params.items() if k.endswith("weight") and "layernorm" not in k]
    nodecay = [v for k, v in params.items() if not (k.endswith("weight") and "layernorm" not in k)]
    norm = torch.nn.utils.clip_grad_norm_(list(params.values()), 1.0)
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": args.weight_decay},
                             {"params": nodecay, "weight_decay": 0.0}], lr=1e-3, betas=(args.adam_beta1, args.adam_beta2),
                            eps=args.adam_eps)
    opt.step()
    # the oracle normalises by the nominal scale only; the matching engine factor is 1 / loss scale
    eng.optimizer.set_grad_factor(1.0)
    ok, grad_norm, _ = eng.optimizer.step(sync=True)
    assert ok and abs(grad_norm - float(norm)) < tol * float(norm), (grad_norm, float(norm))
    for lid, p in eng.stage.named_parameters():
        master = eng.optimizer.state_for_model_parameter(p)["master"].float().cpu()
        after_ref, grad_ref = params[lid].detach(), params[lid].grad
        # The first Adam step moves every element by about lr * sign(g); where g is large compared
        # with the 16-bit noise of the native gradient the two updates must agree closely, and
        # nowhere may they differ by more than one full step in each direction.
        clear = grad_ref.abs() > 0.1 * grad_ref.abs().max()
        assert clear.any()
        assert (master - after_ref)[clear].abs().max() < 1e-4, (lid, float((master - after_ref)[clear].abs().max()))
        assert (master - after_ref).abs().max() < 2.5e-3, (lid, float((master - after_ref).abs().max()))


def test_bounded_device_wait_runs_out_and_reports():
    """A wait for a flag that nothing sets ends by itself after the wait limit: the kernel returns,
    the status word says what gave up, `check_status` raises and resets, and the context keeps
    working. Both 'peers' are local buffers, so nothing faults and nothing else waits."""
    import time
    from eth_b200.ops import native
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    native.check_status(dev)
    mine = torch.zeros(64, dtype=torch.int32, device=dev)
    other = torch.zeros(64, dtype=torch.int32, device=dev)
    t0 = time.time()
    # rank 0 of a "world" of two waits for arrive flags at epoch 1; nobody signals
    native.lib().peer_flags([mine.data_ptr(), other.data_ptr()], 0, 1, -1, 0, native.status(dev))
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 0.5 < waited < 30.0, waited
    assert int(native.status(dev).item()) == 5
    with pytest.raises(RuntimeError, match="peer"):
        native.check_status(dev)
    native.check_status(dev)                       # cleared by the raise above
    x = torch.ones(1024, device=dev)
    assert float((x * 2).sum().item()) == 2048.0   # the context is still usable
    # with the flags set the same call returns at once and leaves the status clean
    mine[:2] = 1
    native.lib().peer_flags([mine.data_ptr(), other.data_ptr()], 0, 1, -1, 0, native.status(dev))
    torch.cuda.synchronize()
    native.check_status(dev)


def test_unfused_attention_ops_on_gpu_match_flash_attention():
    """The four ops of the 13-op manifest (batched tcgen05 GEMMs for Q K^T and P V, the causal
    softmax kernel) against the fused flash-attention kernel: same output, same packed gradient."""
    from eth_b200.ops import native, raw
    dev = torch.device("cuda", 0)
    b, s, heads, d = 2, 256, 4, 64
    torch.manual_seed(0)
    qkv = (torch.randn(b * s, heads * 3 * d, device=dev) * 0.5).to(torch.bfloat16)
    d_out = (torch.randn(b * s, heads * d, device=dev) * 0.5).to(torch.bfloat16)
    out_f, lse = raw.attention_fwd(qkv, b, s, heads, d)
    dqkv_f = raw.attention_bwd(d_out, qkv, out_f, lse, b, s, heads, d)
    scores = raw.attn_scores_fwd(qkv, b, s, heads, d)
    probs = raw.softmax_fwd(scores, d ** -0.5, causal=True)
    out_u = raw.attn_context_fwd(probs, qkv, b, s, heads, d)
    d_probs, dqkv_u = raw.attn_context_bwd(d_out, probs, qkv, b, s, heads, d)
    d_scores = raw.softmax_bwd(d_probs, probs, d ** -0.5, causal=True)
    raw.attn_scores_bwd(d_scores, qkv, dqkv_u, b, s, heads, d)
    torch.cuda.synchronize()
    native.check_status()
    # fp32 reference of the scores, to check the batched GEMM on its own
    v5 = qkv.view(b, s, heads, 3, d).float()
    ref_scores = torch.einsum("bqhd,bkhd->bhqk", v5[:, :, :, 0], v5[:, :, :, 1])
    def err(a, ref):
        a, ref = a.float(), ref.float()
        return max(((a - ref).norm() / ref.norm()).item(), ((a - ref).abs().max() / ref.abs().max()).item())
    assert err(scores, ref_scores) < 1e-2
    assert err(out_u, out_f) < 2e-2
    assert err(dqkv_u, dqkv_f) < 4e-2
