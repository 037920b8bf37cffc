"""Dataset helpers: compiled index builders against their Python restatements; mmap round trip."""
import numpy as np
import pytest

from eth_b200.data import helpers
from eth_b200.data.gpt_dataset import GPTDataset
from eth_b200.data.indexed_dataset import MMapIndexedDataset, MMapIndexedDatasetBuilder
from eth_b200.data.samplers import BlendableDataset, PretrainingSampler
from eth_b200.tokenizer.tokenizer import vocab_size_with_padding


def test_sample_idx_matches_python_oracle():
    rng = np.random.RandomState(0)
    sizes = rng.randint(3, 40, size=50).astype(np.int32)
    doc_idx = np.concatenate([rng.permutation(50) for _ in range(3)]).astype(np.int32)
    tokens = int(sizes.sum())
    ref = helpers.build_sample_idx_python(sizes, doc_idx, 16, 3, tokens)
    got = helpers.build_sample_idx(sizes, doc_idx, 16, 3, tokens)
    assert np.array_equal(np.asarray(got), ref)


def test_blending_follows_weights():
    ds, sample = helpers.build_blending_indices([0.7, 0.2, 0.1], 1000)
    frac = np.bincount(ds, minlength=3) / 1000.0
    assert np.allclose(frac, [0.7, 0.2, 0.1], atol=0.01)
    for k in range(3):
        assert np.array_equal(sample[ds == k], np.arange((ds == k).sum()))


def test_mmap_round_trip_and_gpt_samples(tmp_path):
    prefix = str(tmp_path / "toy")
    b = MMapIndexedDatasetBuilder(prefix + ".bin", dtype=np.uint16)
    docs = [np.arange(i * 10, i * 10 + 7 + i) for i in range(6)]
    for d in docs:
        b.add_item(d)
        b.end_document()
    b.finalize(prefix + ".idx")
    ds = MMapIndexedDataset(prefix)
    assert len(ds) == 6 and np.array_equal(ds[3], docs[3])
    gpt = GPTDataset(ds, np.arange(6), num_samples=8, seq_length=5, seed=1)
    assert len(gpt) >= 8
    for i in range(len(gpt)):
        assert gpt[i]["text"].shape == (6,)


def test_sampler_shards_batches():
    a = list(PretrainingSampler(20, 4, 2, 0, 2))
    b = list(PretrainingSampler(20, 4, 2, 1, 2))
    assert a[0] == [4, 5] and b[0] == [6, 7] and len(a) == 4


def test_blendable_dataset():
    d = BlendableDataset([list(range(10)), list(range(100, 130))], [0.25, 0.75])
    assert len(d) == 40 and all(isinstance(d[i], int) for i in range(40))


@pytest.mark.parametrize("tp,expected", [(1, 50304), (2, 50432), (4, 50688)])
def test_vocab_padding(tp, expected):
    assert vocab_size_with_padding(50257, 128, tp) == expected


# ------------------------------------------------------------------ dataset -> engine input path
def _toy_dataset(tmp_path, name="toy", n_docs=40, vocab=60, seed=0):
    prefix = str(tmp_path / name)
    rng = np.random.RandomState(seed)
    b = MMapIndexedDatasetBuilder(prefix + ".bin", dtype=np.uint16)
    for _ in range(n_docs):
        b.add_item(rng.randint(1, vocab, size=rng.randint(5, 30)))
        b.end_document()
    b.finalize(prefix + ".idx")
    return prefix


def test_split_offsets_cover_all_documents():
    from eth_b200.data.provider import split_offsets
    assert split_offsets("949,50,1", 1000) == [0, 949, 999, 1000]
    assert split_offsets("98/2", 50) == [0, 49, 50, 50]
    assert split_offsets("1", 7) == [0, 7, 7, 7]
    edges = split_offsets("1,1,1", 10)
    assert edges[0] == 0 and edges[-1] == 10 and edges == sorted(edges)
    with pytest.raises(ValueError):
        split_offsets("0,0,0", 10)


def test_last_epoch_is_shuffled_apart_when_mostly_unused(tmp_path):
    """A run that needs a small part of its last epoch keeps that epoch out of the global shuffle:
    the first `samples before the last epoch` draws then cover exactly the full epochs."""
    from eth_b200.data.gpt_dataset import last_epoch_is_separate, num_tokens_per_epoch
    ds = MMapIndexedDataset(_toy_dataset(tmp_path))
    docs = np.arange(len(ds.sizes), dtype=np.int32)
    tokens, seq = num_tokens_per_epoch(ds.sizes, docs), 8
    per_epoch = (tokens - 1) // seq
    want = 2 * per_epoch + 3                      # two full epochs and a sliver of the third
    gpt = GPTDataset(ds, docs, num_samples=want, seq_length=seq, seed=3)
    separate, before = last_epoch_is_separate(tokens, seq, want, 3)
    assert separate and gpt.separate_last_epoch
    head = np.sort(np.asarray(gpt.shuffle_idx[:before]))
    assert np.array_equal(head, np.arange(before))
    # most of the last epoch is needed: one shuffle over everything
    full = GPTDataset(ds, docs, num_samples=3 * per_epoch - 2, seq_length=seq, seed=3)
    assert not full.separate_last_epoch
    assert last_epoch_is_separate(tokens, seq, per_epoch - 1, 1) == (False, 0)


def test_dataset_provider_shifts_labels_and_masks_eod(tmp_path):
    from eth_b200.data.provider import DatasetProvider, build_datasets
    prefix = _toy_dataset(tmp_path)
    train, valid, test = build_datasets([prefix], "8,1,1", (64, 8, 8), seq_length=12, seed=5)
    assert train is not None and valid is not None and test is not None
    eod = 7
    prov = DatasetProvider(train, eod_token=eod, eod_mask_loss=True)
    tokens, labels, mask = prov([0, 1, 2], 12, "cpu")
    assert tokens.shape == labels.shape == mask.shape == (3, 12)
    assert np.array_equal(tokens[:, 1:].numpy(), labels[:, :-1].numpy())
    assert np.array_equal(np.concatenate([tokens[0].numpy(), labels[0, -1:].numpy()]), train[0]["text"])
    assert np.array_equal(mask.numpy() == 0, tokens.numpy() == eod)
    # a shorter micro-batch sequence takes the head of the sample; ids wrap around the dataset
    t2, l2, _ = prov([len(train)], 6, "cpu")
    assert np.array_equal(t2[0].numpy(), train[0]["text"][:6]) and l2[0, -1] == train[0]["text"][6]
    # weight/prefix pairs blend
    other = _toy_dataset(tmp_path, "other", seed=9)
    blend, _, _ = build_datasets(["0.3", prefix, "0.7", other], "1,0,0", (50, 0, 0), seq_length=12, seed=5)
    assert len(blend) >= 50 and blend[0]["text"].shape == (13,)


def test_pretrain_reads_indexed_dataset(tmp_path, capsys):
    """`--data-path` reaches the engine: training consumes dataset tokens (not the synthetic formula)
    and evaluation reads the validation part from its own cursor."""
    import json
    from eth_b200.contract.config import uniform_config
    from eth_b200.runtime.pretrain_gpt import pretrain
    prefix = _toy_dataset(tmp_path, n_docs=80)
    model = dict(model_size="tiny", num_layers=2, hidden_size=32, num_attention_heads=4, seq_length=16,
                 max_position_embeddings=16)
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(uniform_config(model, pp=1, tp=1, dp=1, gbs=4, mbs=2)))
    seen = []
    from eth_b200.data import provider as provider_mod
    original = provider_mod.DatasetProvider.host_batch

    def spy(self, ids, seq):
        out = original(self, ids, seq)
        seen.append((self, list(ids), out[0].copy()))
        return out
    provider_mod.DatasetProvider.host_batch = spy
    try:
        engine = pretrain(["--flexpipe-config", str(cfg_path), "--device", "cpu", "--vocab-size", "64",
                           "--make-vocab-size-divisible-by", "8", "--train-iters", "2", "--eval-iters", "1",
                           "--eval-interval", "2", "--hidden-dropout", "0.0", "--data-path", prefix,
                           "--split", "8,2,0", "--lr", "1e-3"])
    finally:
        provider_mod.DatasetProvider.host_batch = original
    out = capsys.readouterr().out
    assert "validation loss at iteration 2" in out and "validation set: yes" in out
    train_calls = [c for c in seen if c[0] is engine.data_provider]
    eval_calls = [c for c in seen if c[0] is engine.eval_data_provider]
    assert [c[1] for c in train_calls] == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert [c[1] for c in eval_calls] == [[0, 1], [2, 3]] and engine.eval_cursor == 4
    assert engine.clock.global_data_cursor == 8
    assert np.array_equal(train_calls[0][2][0], engine.data_provider.dataset[0]["text"][:16])
