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
