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
