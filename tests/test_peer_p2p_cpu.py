"""Peer-memory pipeline transfers, host side: the copy descriptors of every sender, applied to byte
arrays that stand for the receivers' ring slots, deliver to every receiver exactly its shard of the
logical tensor, for equal and for changing TP x DP layouts across a stage boundary."""
import numpy as np
import pytest
import torch

from eth_b200.contract.config import make_config, make_pipe, manifest_size, normalize_flexpipe_config
from eth_b200.models.gpt_ops import LIVE_AFTER
from eth_b200.parallel.grad_sync.topology import build_canonical_topology
from eth_b200.parallel.p2p import plan_transfers
from eth_b200.parallel.peer_p2p import Direction, slot_layout

LAYERS, HIDDEN, SEQ, MBS = 2, 32, 8, 4


def _stages(tp, dp, cut):
    n = manifest_size(LAYERS)
    cfg = make_config([make_pipe([cut, n - cut], list(tp), list(dp), gbs=8, mbs=MBS)], num_layers=LAYERS,
                      hidden_size=HIDDEN, num_attention_heads=4, seq_length=SEQ)
    topo = build_canonical_topology(normalize_flexpipe_config(cfg))
    return topo.stage(0, 0), topo.stage(0, 1)


def _shard(full, stage, coord, spec_entry):
    """What `coord` of `stage` holds of the logical tensor `full` ([MBS * SEQ, features] or [features])."""
    _, mult, sharded, per_token = spec_entry
    feat = mult * HIDDEN
    cols = slice(coord.tp_rank * feat // stage.tp_degree, (coord.tp_rank + 1) * feat // stage.tp_degree) if sharded \
        else slice(0, feat)
    if not per_token:
        return full[cols]
    b = MBS // stage.dp_degree
    return full[coord.dp_rank * b * SEQ:(coord.dp_rank + 1) * b * SEQ, cols]


@pytest.mark.parametrize("tp,dp,cut,after", [
    ((1, 1), (1, 1), 11, "enc-post-MLP-dropout"),        # layer boundary, same shape
    ((2, 2), (1, 1), 3, "enc-attention-qkv"),            # mid-layer: TP-sharded qkv + residual
    ((2, 1), (1, 2), 11, "enc-post-MLP-dropout"),        # TP2 -> DP2
    ((1, 2), (2, 1), 4, "enc-flash-attention"),          # DP2 -> TP2 with a sharded tensor
    ((2, 2), (2, 2), 6, "enc-attention-dense"),          # hidden + bias vector + residual
])
@pytest.mark.parametrize("grads", [False, True])
def test_copy_descriptors_deliver_every_receivers_shard(tp, dp, cut, after, grads):
    first, second = _stages(tp, dp, cut)
    spec = LIVE_AFTER[after]
    src_stage, dst_stage = (second, first) if grads else (first, second)
    dtype = torch.float32                       # exact comparison; element sizes are what matters
    rng = np.random.RandomState(0)
    logical = {}
    for name, mult, sharded, per_token in spec:
        shape = (MBS * SEQ, mult * HIDDEN) if per_token else (mult * HIDDEN,)
        logical[name] = rng.randn(*shape).astype(np.float32)
    pieces = plan_transfers(src_stage, dst_stage, spec, MBS, HIDDEN)
    inbox = {}
    layout = None
    for coord in src_stage.rank_coordinates:
        d = Direction(coord.global_rank, pieces, spec, SEQ, HIDDEN, dtype, grads, src_stage, dst_stage, MBS)
        layout = d.dst_layout
        for c in d.copies:
            entry = next(e for e in spec if e[0] == c.name)
            src = np.ascontiguousarray(_shard(logical[c.name], src_stage, coord, entry)).view(np.uint8).reshape(-1)
            box = inbox.setdefault(c.dst_rank, np.zeros(d.slot_bytes, dtype=np.uint8))
            for row in range(c.rows):
                a, b = c.src_offset + row * c.src_pitch, c.dst_offset + row * c.dst_pitch
                box[b:b + c.width] = src[a:a + c.width]
        # every receiver knows which ranks write to it, and each writer has its own flag
        for dst, writers in d.writers.items():
            assert writers == sorted(set(writers)) and len(writers) <= 16
    assert set(inbox) == {c.global_rank for c in dst_stage.rank_coordinates}
    for coord in dst_stage.rank_coordinates:
        tokens = MBS // dst_stage.dp_degree * SEQ
        mine, size = slot_layout(spec, tokens, HIDDEN, dst_stage.tp_degree, dtype, grads)
        assert [(t.name, t.shape, t.offset) for t in mine] == [(t.name, t.shape, t.offset) for t in layout]
        for t in mine:
            entry = next(e for e in spec if e[0] == t.name)
            got = inbox[coord.global_rank][t.offset:t.offset + t.nbytes].view(np.float32).reshape(t.shape)
            assert np.array_equal(got, _shard(logical[t.name], dst_stage, coord, entry)), (t.name, coord)


def test_gradient_vectors_travel_in_fp32():
    spec = LIVE_AFTER["enc-attention-dense"]
    acts, _ = slot_layout(spec, 16, HIDDEN, 1, torch.bfloat16, grads=False)
    grads, _ = slot_layout(spec, 16, HIDDEN, 1, torch.bfloat16, grads=True)
    by = {t.name: t.dtype for t in grads}
    assert by["output_bias"] == torch.float32 and by["hidden_states"] == torch.bfloat16
    assert all(t.dtype == torch.bfloat16 for t in acts)
    assert all(t.offset % 256 == 0 for t in acts + grads)
