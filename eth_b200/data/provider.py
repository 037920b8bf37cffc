"""Batches for the training engine from indexed token files, or built on the host from the
synthetic formula.

The engine asks a provider for the samples of one micro-batch by their global sample ids
(`provider(sample_ids, seq, device) -> tokens, labels, loss_mask`); which ids a rank gets follows
from the training clock and the sample schedule, the role the batch sampler with its
`consumed_samples` plays in the reference (eth/runtime/megatron/data/data_samplers.py:57-104). This
module covers the rest of the reference's input path: the document split and the train / valid /
test datasets with blending (data/gpt_dataset.py:31-140, dataset_utils.py:51-69), the sample counts
(eth/runtime/pretrain_gpt.py:139-160 via training.py:1535-1560), tokens/labels/mask from a
`seq + 1` token sample (pretrain_gpt.py:60-96, utils.py:143-194) and the broadcast from the first
rank of a tensor-parallel group (mpu/data.py:76-117). Every batch is staged in pinned host memory
and copied with non-blocking copies; a small ring of staging buffers keeps the host one or two
micro-batches ahead of the device.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .gpt_dataset import GPTDataset
from .indexed_dataset import make_dataset
from .samplers import BlendableDataset


# ------------------------------------------------------------------------------------------ splits
def split_offsets(splits: str, size: int) -> List[int]:
    """Document offsets [0, a, b, size] of the train / valid / test parts for a proportion string
    such as "949,50,1" or "98/2"."""
    sep = "," if "," in splits else "/"
    parts = [float(v) for v in splits.split(sep) if v.strip()][:3]
    parts += [0.0] * (3 - len(parts))
    total = sum(parts)
    if total <= 0:
        raise ValueError(f"--split {splits!r} has no positive part")
    edges = [0]
    for share in parts:
        edges.append(edges[-1] + int(round(share / total * size)))
    excess = edges[-1] - size   # rounding: shift every edge so the last one lands on `size`
    return [0] + [e - excess for e in edges[1:]]


def parse_data_path(data_path: Sequence[str]) -> Tuple[List[float], List[str]]:
    """`[prefix]` or `[w0, prefix0, w1, prefix1, ...]` -> (normalised weights, prefixes)."""
    items = list(data_path)
    if len(items) == 1:
        return [1.0], items
    if len(items) % 2:
        raise ValueError("--data-path takes one prefix, or weight/prefix pairs")
    weights = [float(w) for w in items[0::2]]
    total = sum(weights)
    if total <= 0:
        raise ValueError("--data-path weights must sum to a positive value")
    return [w / total for w in weights], items[1::2]


def sample_counts(train_iters: int, global_batch: int, eval_interval: int, eval_iters: int) -> Tuple[int, int, int]:
    """Samples needed from the train / valid / test datasets over the whole run."""
    evals = (train_iters // eval_interval + 1) * eval_iters if eval_interval and eval_iters else 0
    return train_iters * global_batch, evals * global_batch, eval_iters * global_batch


def build_datasets(data_path: Sequence[str], splits: str, counts: Sequence[int], seq_length: int, seed: int,
                   data_impl: str = "mmap"):
    """(train, valid, test) datasets; a part whose split share is empty is None. With several
    prefixes each part is a weighted blend and every member is built for its share of the samples
    (plus the reference's 0.5 % margin, so a blend never runs a member dry)."""
    weights, prefixes = parse_data_path(data_path)
    per_prefix = []
    for weight, prefix in zip(weights, prefixes):
        indexed = make_dataset(prefix, data_impl)
        edges = split_offsets(splits, len(indexed.sizes))
        need = [int(np.ceil(n * weight * 1.005)) if len(prefixes) > 1 else int(n) for n in counts]
        parts = []
        for k in range(3):
            if edges[k + 1] > edges[k] and need[k] > 0:
                docs = np.arange(edges[k], edges[k + 1], dtype=np.int32)
                parts.append(GPTDataset(indexed, docs, need[k], seq_length, seed))
            else:
                parts.append(None)
        per_prefix.append(parts)
    if len(prefixes) == 1:
        return tuple(per_prefix[0])
    out = []
    for k in range(3):
        members = [(p[k], w) for p, w in zip(per_prefix, weights) if p[k] is not None]
        out.append(BlendableDataset([m for m, _ in members], [w for _, w in members]) if members else None)
    return tuple(out)


# ------------------------------------------------------------------------------------------ staging
class _PinnedRing:
    """A few pinned (tokens, labels, mask) triples per batch shape, reused round-robin; a triple is
    handed out again only after the copies that last read it have finished."""

    def __init__(self, depth: int = 4):
        self.depth, self.slots, self.events, self.cursor = depth, {}, {}, 0
        self.h2d_bytes = 0

    def stage(self, tokens: np.ndarray, labels: np.ndarray, mask: np.ndarray, device):
        device = torch.device(device)
        if device.type != "cuda":
            return torch.from_numpy(tokens).clone(), torch.from_numpy(labels).clone(), torch.from_numpy(mask).clone()
        key = (tokens.shape, self.cursor % self.depth)
        self.cursor += 1
        if key not in self.slots:
            self.slots[key] = (torch.empty(tokens.shape, dtype=torch.long).pin_memory(),
                               torch.empty(tokens.shape, dtype=torch.long).pin_memory(),
                               torch.empty(tokens.shape, dtype=torch.float32).pin_memory())
        else:
            self.events[key].synchronize()
        pt, pl, pm = self.slots[key]
        pt.copy_(torch.from_numpy(tokens))
        pl.copy_(torch.from_numpy(labels))
        pm.copy_(torch.from_numpy(mask))
        out = (pt.to(device, non_blocking=True), pl.to(device, non_blocking=True), pm.to(device, non_blocking=True))
        done = torch.cuda.Event()
        done.record()
        self.events[key] = done
        self.h2d_bytes += pt.numel() * 8 + pl.numel() * 8 + pm.numel() * 4
        return out


class SyntheticHostProvider:
    """The synthetic batch formula evaluated on the host (numpy) and copied from pinned memory: the
    same tokens as the device-side generator, through the input path a real dataset takes."""

    def __init__(self, vocab: int):
        self.vocab, self.ring = int(vocab), _PinnedRing()

    @property
    def h2d_bytes(self) -> int:
        return self.ring.h2d_bytes

    def reset_counter(self) -> None:
        self.ring.h2d_bytes = 0

    def __call__(self, sample_ids, seq, device):
        ids = np.asarray(sample_ids, dtype=np.int64)[:, None]
        pos = np.arange(seq, dtype=np.int64)[None, :]
        tokens = (ids * 1103515245 + pos * 12345) % self.vocab
        labels = (ids * 1103515245 + (pos + 1) * 12345) % self.vocab
        mask = ((ids + pos) % 4 != 0).astype(np.float32)
        return self.ring.stage(tokens, labels, mask, device)


class DatasetProvider:
    """Micro-batches from a GPT dataset: sample `i` is `seq + 1` tokens; tokens are its first `seq`,
    labels the same shifted by one, and the loss mask is one everywhere, or zero on end-of-document
    tokens with `eod_mask_loss`. A sequence shorter than the dataset's (variable-length micro-batch
    plans) takes the head of the sample."""

    def __init__(self, dataset, eod_token: Optional[int] = None, eod_mask_loss: bool = False):
        if dataset is None or len(dataset) == 0:
            raise ValueError("the dataset for this phase is empty (check --split)")
        self.dataset, self.eod, self.eod_mask_loss = dataset, eod_token, eod_mask_loss
        self.ring = _PinnedRing()

    def host_batch(self, sample_ids, seq: int):
        n = len(self.dataset)
        rows = []
        for i in sample_ids:
            text = self.dataset[int(i) % n]["text"]
            if text.shape[0] < seq + 1:
                raise ValueError(f"sample {int(i)} has {text.shape[0]} tokens, {seq + 1} are needed")
            rows.append(text[:seq + 1])
        block = np.stack(rows).astype(np.int64)
        tokens, labels = np.ascontiguousarray(block[:, :-1]), np.ascontiguousarray(block[:, 1:])
        mask = np.ones(tokens.shape, dtype=np.float32)
        if self.eod_mask_loss and self.eod is not None:
            mask[tokens == self.eod] = 0.0
        return tokens, labels, mask

    def __call__(self, sample_ids, seq, device):
        return self.ring.stage(*self.host_batch(sample_ids, seq), device)


class TensorParallelFeed:
    """Only the first rank of a tensor-parallel group reads the data; its peers receive tokens,
    labels and mask (as int64) through `broadcast_data`: shapes, then one flat payload."""
    KEYS = ("tokens", "labels", "mask")

    def __init__(self, inner: Optional[Callable], src_rank: int, group, is_source: bool):
        self.inner, self.src, self.group, self.is_source = inner, src_rank, group, is_source

    def __call__(self, sample_ids, seq, device):
        from ..parallel.data_broadcast import broadcast_data
        data = None
        if self.is_source:
            tokens, labels, mask = self.inner(sample_ids, seq, device)
            data = {"tokens": tokens, "labels": labels, "mask": mask.to(torch.long)}
        out = broadcast_data(self.KEYS, data, torch.long, self.src, group=self.group, device=torch.device(device))
        return out["tokens"], out["labels"], out["mask"].to(torch.float32)


def providers_from_args(args, pstate, eod_token: Optional[int] = None):
    """(train provider, validation provider) for this rank as the flags ask: indexed datasets with
    `--data-path`, host-built synthetic batches with `--host-data`, else (None, None) and the engine
    generates synthetic batches on the device."""
    if getattr(args, "data_path", None):
        is_source = pstate.tp_rank == 0
        train = valid = None
        if is_source or pstate.tp_size == 1:
            counts = sample_counts(args.train_iters, args.total_gbs, args.eval_interval, args.eval_iters)
            ds_train, ds_valid, _ = build_datasets(args.data_path, args.split, counts, args.seq_length, args.seed,
                                                   args.data_impl)
            mask_eod = bool(getattr(args, "eod_mask_loss", False))
            train = DatasetProvider(ds_train, eod_token, mask_eod)
            valid = DatasetProvider(ds_valid, eod_token, mask_eod) if ds_valid is not None else None
        if pstate.tp_size > 1:
            src = pstate.tp_group_ranks[0]
            has_valid = [valid is not None]
            if getattr(pstate, "tp_group", None) is not None:
                import torch.distributed as dist
                dist.broadcast_object_list(has_valid, src, group=pstate.tp_group)
            train = TensorParallelFeed(train, src, pstate.tp_group, is_source)
            valid = TensorParallelFeed(valid, src, pstate.tp_group, is_source) if has_valid[0] else None
        return train, valid
    if getattr(args, "host_data", False):
        provider = SyntheticHostProvider(args.vocab_size)
        return provider, provider
    return None, None
