"""Batch samplers that resume from `consumed_samples` and shard a global batch over data-parallel
ranks (reference: eth/runtime/megatron/data/data_samplers.py:57-157), plus dataset blending
(blendable_dataset.py:27-68)."""
from __future__ import annotations

import numpy as np

from .helpers import build_blending_indices


class PretrainingSampler:
    def __init__(self, total_samples, consumed_samples, micro_batch_size, data_parallel_rank, data_parallel_size,
                 drop_last=True):
        if total_samples <= 0 or consumed_samples >= total_samples:
            raise ValueError("no samples left to consume")
        if micro_batch_size <= 0 or not 0 <= data_parallel_rank < data_parallel_size:
            raise ValueError("invalid sampler shape")
        self.total, self.consumed = total_samples, consumed_samples
        self.mbs, self.rank, self.size, self.drop_last = micro_batch_size, data_parallel_rank, data_parallel_size, drop_last
        self.step = micro_batch_size * data_parallel_size

    def __len__(self):
        return self.total

    def __iter__(self):
        batch = []
        lo = self.rank * self.mbs
        for idx in range(self.consumed, self.total):
            batch.append(idx)
            if len(batch) == self.step:
                yield batch[lo:lo + self.mbs]
                batch = []
        if batch and not self.drop_last:
            yield batch[lo:lo + self.mbs]


class PretrainingRandomSampler(PretrainingSampler):
    def __iter__(self):
        active = self.total - self.total % self.step
        epoch = self.consumed // active
        done = self.consumed % active
        bucket = (self.total // self.step) * self.mbs
        offset = done // self.size
        start = self.rank * bucket
        rng = np.random.RandomState(epoch)
        order = (start + rng.permutation(bucket))[offset:]
        batch = []
        for idx in order.tolist():
            batch.append(idx)
            if len(batch) == self.mbs:
                self.consumed += self.step
                yield batch
                batch = []


class BlendableDataset:
    def __init__(self, datasets, weights):
        if len(datasets) != len(weights) or not datasets:
            raise ValueError("one weight per dataset is required")
        w = np.asarray(weights, dtype=np.float64)
        if w.sum() <= 0:
            raise ValueError("weights must sum to a positive value")
        self.datasets = datasets
        self.size = sum(len(d) for d in datasets)
        self.dataset_index, self.dataset_sample_index = build_blending_indices(w / w.sum(), self.size)

    def __len__(self):
        return self.size

    def __getitem__(self, idx):
        d = int(self.dataset_index[idx])
        return self.datasets[d][int(self.dataset_sample_index[idx]) % len(self.datasets[d])]
