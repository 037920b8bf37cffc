"""GPT dataset over an indexed token file: document, sample and shuffle indices
(reference: eth/runtime/megatron/data/gpt_dataset.py:190-325 index building, :364-410 the Python
sample-index oracle). Sample i is the `seq_length + 1` tokens starting at
`sample_idx[shuffle_idx[i]]`, crossing document boundaries as needed."""
from __future__ import annotations

import numpy as np

from .helpers import build_sample_idx


def num_tokens_per_epoch(sizes, documents) -> int:
    return int(np.sum(sizes[documents]))


def num_epochs_for(tokens_per_epoch: int, seq_length: int, num_samples: int) -> int:
    epochs, total = 0, 0
    while True:
        epochs += 1
        total += tokens_per_epoch
        if (total - 1) // seq_length >= num_samples:
            return epochs


def build_doc_idx(documents, num_epochs: int, rng: np.random.RandomState, separate_last_epoch: bool = False):
    if not separate_last_epoch or num_epochs == 1:
        doc_idx = np.mgrid[0:num_epochs, 0:len(documents)][1]
        doc_idx[:] = documents
        doc_idx = doc_idx.reshape(-1).astype(np.int32)
        rng.shuffle(doc_idx)
        return doc_idx
    first = build_doc_idx(documents, num_epochs - 1, rng, False)
    last = build_doc_idx(documents, 1, rng, False)
    return np.concatenate((first, last))


def build_shuffle_idx(num_samples: int, total_size: int, rng: np.random.RandomState):
    dtype = np.uint32 if total_size < np.iinfo(np.uint32).max - 1 else np.int64
    first = np.arange(0, num_samples, dtype=dtype)
    rng.shuffle(first)
    if num_samples == total_size:
        return first
    last = np.arange(num_samples, total_size, dtype=dtype)
    rng.shuffle(last)
    return np.concatenate((first, last))


def last_epoch_is_separate(tokens_per_epoch: int, seq_length: int, num_samples: int, epochs: int):
    """(separate, samples before the last epoch). When the run needs only a small part (< 80 %) of
    its last epoch, that epoch's samples must not be mixed into the global shuffle: they would push
    samples of the full epochs out of the first `num_samples` draws. The last epoch then gets its
    own document order and its own shuffle range (reference: gpt_dataset.py:222-262, 286-293)."""
    if epochs == 1:
        return False, 0
    before = ((epochs - 1) * tokens_per_epoch - 1) // seq_length
    in_last = num_samples - before
    per_epoch = (tokens_per_epoch - 1) // seq_length
    if not 0 <= in_last <= per_epoch:
        raise ValueError(f"inconsistent epoch arithmetic: {in_last} samples in the last epoch of {per_epoch}")
    return in_last < int(0.80 * per_epoch), before


class GPTDataset:
    """Index maps are built in memory on every rank from (documents, num_samples, seq_length, seed):
    deterministic, so ranks agree without the reference's .npy files beside the data."""

    def __init__(self, indexed_dataset, documents, num_samples: int, seq_length: int, seed: int):
        self.data, self.seq_length = indexed_dataset, seq_length
        documents = np.asarray(documents, dtype=np.int32)
        tokens = num_tokens_per_epoch(indexed_dataset.sizes, documents)
        epochs = num_epochs_for(tokens, seq_length, num_samples)
        rng = np.random.RandomState(seed)
        separate, before_last = last_epoch_is_separate(tokens, seq_length, num_samples, epochs)
        self.separate_last_epoch = separate
        self.doc_idx = build_doc_idx(documents, epochs, rng, separate)
        self.sample_idx = build_sample_idx(np.asarray(indexed_dataset.sizes, dtype=np.int32), self.doc_idx, seq_length,
                                           epochs, tokens)
        n = self.sample_idx.shape[0] - 1
        self.shuffle_idx = build_shuffle_idx(before_last if separate else n, n, rng)

    def __len__(self) -> int:
        return self.sample_idx.shape[0] - 1

    def __getitem__(self, idx: int):
        idx = int(self.shuffle_idx[idx])
        d0, o0 = self.sample_idx[idx]
        d1, o1 = self.sample_idx[idx + 1]
        if d0 == d1:
            sample = self.data.get(int(self.doc_idx[d0]), offset=int(o0), length=int(o1 - o0 + 1))
        else:
            parts = [self.data.get(int(self.doc_idx[d0]), offset=int(o0))]
            parts += [self.data.get(int(self.doc_idx[d])) for d in range(d0 + 1, d1)]
            parts.append(self.data.get(int(self.doc_idx[d1]), length=int(o1 + 1)))
            sample = np.concatenate(parts)
        return {"text": np.asarray(sample, dtype=np.int64)}
