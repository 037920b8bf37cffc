"""Memory buffers, TP data broadcast and forward-only evaluation (CPU)."""
import pytest
import torch

from eth_b200.utils import memory
from tests.helpers.multiproc import run_ranks


def test_memory_buffer_and_ring():
    buf = memory.MemoryBuffer("t", 100, torch.float32, track_usage=True, device="cpu")
    a = buf.add(torch.arange(12, dtype=torch.float32).view(3, 4))
    b = buf.view((5, 2))
    assert a.data_ptr() == buf.data.data_ptr() and b.data_ptr() == buf.data[12:].data_ptr()
    assert buf.numel_in_use() == 22 and buf.get_data().numel() == 22
    with pytest.raises(MemoryError):
        buf.view((100,))
    with pytest.raises(TypeError):
        buf.add(torch.zeros(2, dtype=torch.float16))
    buf.reset()
    assert not buf.is_in_use()
    ring = memory.RingMemBuffer("ring-test", 2, 16, torch.float32, device="cpu")
    first = ring.get_next_buffer()
    first.view((4,))
    second = ring.get_next_buffer()
    assert second is not first
    with pytest.raises(RuntimeError):
        ring.get_next_buffer()
    first.reset()
    assert ring.get_next_buffer() is first
    for i in range(2):
        memory.free_mem_buff(f"ring-test {i}")


def _bcast(rank, world):
    from eth_b200.parallel.data_broadcast import broadcast_data
    data = None
    if rank == 0:
        data = {"text": torch.arange(24).view(2, 12), "labels": torch.arange(6).view(2, 3) + 100}
    out = broadcast_data(["text", "labels"], data, torch.int64, src=0)
    return out["text"].tolist(), out["labels"].tolist()


def test_broadcast_data():
    res = run_ranks(2, _bcast)
    assert res[0] == res[1]
    assert res[1][0] == torch.arange(24).view(2, 12).tolist()


def test_eval_step_leaves_training_state_alone():
    from eth_b200.contract.config import uniform_config
    from eth_b200.runtime.arguments import parse_args
    from eth_b200.runtime.engine import TrainEngine
    from eth_b200.runtime.pretrain_gpt import evaluate
    model = dict(model_size="tiny", num_layers=2, hidden_size=64, num_attention_heads=4, seq_length=32,
                 max_position_embeddings=32)
    config = uniform_config(model, pp=1, tp=1, dp=1, gbs=4, mbs=2)
    args = parse_args(["--vocab-size", "128", "--train-iters", "2", "--hidden-dropout", "0.1"], config=config,
                      rank=0, world_size=1, local_rank=0)
    eng = TrainEngine(args, device=torch.device("cpu"))
    eng.train_step()
    params = eng.stage.param_buf.clone()
    cursor, it = eng.clock.global_data_cursor, eng.iteration
    r1 = evaluate(eng, 2)
    r2 = evaluate(eng, 2)
    assert r1["lm loss"] == r2["lm loss"] and r1["lm loss"] > 0        # dropout off -> deterministic
    assert torch.equal(params, eng.stage.param_buf)
    assert (eng.clock.global_data_cursor, eng.iteration) == (cursor, it)
    assert not eng.stage._contexts


def test_unfused_attention_matches_reference_on_cpu():
    from eth_b200.ops import functional as Fn
    torch.manual_seed(3)
    q, k, v = (torch.randn(2, 24, 3, 16) for _ in range(3))
    for causal in (True, False):
        got = Fn.unfused_attention(q, k, v, causal=causal)
        ref = Fn.attention_ref(q, k, v, 16 ** -0.5, causal)
        torch.testing.assert_close(got, ref, rtol=1e-5, atol=1e-5)
    dropped = Fn.unfused_attention(q, k, v, dropout_p=0.5, seed=1, offset=2)
    assert dropped.shape == q.shape and not torch.equal(dropped, Fn.unfused_attention(q, k, v))
