"""Global loss normalisation, sample ownership and the training clock.

Contract (reference: eth/runtime/megatron/grad_sync/loss.py):
  * Loss. A forward step yields a masked loss *sum* and the mask *weight*; what is back-propagated
    is `loss_sum / nominal`, where `nominal` is a constant of the config (sum over all micro-batches
    of samples x sequence length). After the last micro-batch the gradients are multiplied by
    `nominal / (weight summed over the world)`, which turns the sum into the mean over the tokens
    that actually counted (:33-39).
  * Samples. One global cursor numbers all samples ever drawn. Within a global batch, pipeline p
    starts at its offset, micro-batch m after the micro-batches before it, and data-parallel rank
    d takes the d-th equal part of the micro-batch (:70-97). `SampleSchedule` holds the prefix sums.
  * Synthetic data is a closed formula of (sample id, position) (:100-119), so any rank can build
    its part without I/O.
  * Clock. The cursor advances on every attempted step, the step counter only on success, so an
    overflow-skipped iteration consumes data but not schedule (:122-137).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from itertools import accumulate
from typing import List, Sequence, Tuple

import torch

SYNTH_MUL, SYNTH_POS = 1103515245, 12345


# ------------------------------------------------------------------------------------------
# loss
# ------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class LossOutput:
    local_loss_sum: object
    local_loss_weight: object
    nominal_global_loss_scale: float
    metrics: dict = field(default_factory=dict)


def _positive(value, what):
    if not value > 0:
        raise ValueError(f"{what} must be positive")
    return value


def gpt_loss_output(losses, loss_mask, nominal_global_loss_scale, metrics=None) -> LossOutput:
    _positive(nominal_global_loss_scale, "nominal_global_loss_scale")
    per_token, weight = losses.float().reshape(-1), loss_mask.float().reshape(-1)
    if per_token.shape != weight.shape:
        raise ValueError("GPT loss and loss_mask must have the same numel")
    return LossOutput(torch.dot(per_token, weight), weight.sum(), float(nominal_global_loss_scale), metrics or {})


def global_normalization_scale(nominal_global_loss_scale, global_loss_weight):
    _positive(nominal_global_loss_scale, "nominal_global_loss_scale")
    _positive(float(global_loss_weight.detach().item()), "global_loss_weight")
    return nominal_global_loss_scale / global_loss_weight


def sum_loss_outputs(outputs) -> Tuple[object, object]:
    outputs = list(outputs)
    if not outputs:
        raise ValueError("loss_outputs must not be empty")
    total, weight = outputs[0].local_loss_sum, outputs[0].local_loss_weight
    for o in outputs[1:]:
        total, weight = total + o.local_loss_sum, weight + o.local_loss_weight
    return total, weight


# ------------------------------------------------------------------------------------------
# sample ownership
# ------------------------------------------------------------------------------------------
class SampleSchedule:
    """Where each (pipeline, micro-batch, data-parallel rank) finds its samples inside a global batch."""

    def __init__(self, mbs_sequences: Sequence, pipeline_sample_offsets: Sequence[int]):
        self.sizes: List[List[int]] = [[int(item[0]) for item in seq] for seq in mbs_sequences]
        self.starts: List[List[int]] = [[0] + list(accumulate(sz))[:-1] for sz in self.sizes]
        self.offsets = list(pipeline_sample_offsets)

    def slots(self, pipeline_id: int, microbatch: int, dp_degree: int, dp_rank: int, cursor: int) -> Tuple[int, ...]:
        if not 0 <= pipeline_id < len(self.sizes):
            raise ValueError(f"unknown pipeline_id {pipeline_id}")
        if not 0 <= microbatch < len(self.sizes[pipeline_id]):
            raise ValueError(f"unknown microbatch_index {microbatch}")
        if dp_degree <= 0 or not 0 <= dp_rank < dp_degree:
            raise ValueError("invalid DP coordinate")
        share, rest = divmod(self.sizes[pipeline_id][microbatch], dp_degree)
        if rest:
            raise ValueError("global microbatch size must be divisible by DP degree")
        first = cursor + self.offsets[pipeline_id] + self.starts[pipeline_id][microbatch] + dp_rank * share
        return tuple(range(first, first + share))


def local_sample_slots(pipeline_id: int, microbatch_index: int, dp_degree: int, dp_rank: int,
                       mbs_sequences: Sequence, pipeline_sample_offsets: Sequence[int], global_data_cursor: int):
    return SampleSchedule(mbs_sequences, pipeline_sample_offsets).slots(pipeline_id, microbatch_index, dp_degree,
                                                                        dp_rank, global_data_cursor)


# ------------------------------------------------------------------------------------------
# synthetic data
# ------------------------------------------------------------------------------------------
def _ids_on_device(sample_ids, device) -> torch.Tensor:
    if isinstance(sample_ids, torch.Tensor):
        return sample_ids.to(device=device, dtype=torch.long)
    ids = tuple(sample_ids)
    if ids and ids[-1] - ids[0] == len(ids) - 1:
        # consecutive slots: generate them on the device (copying from the host would synchronise)
        return torch.arange(ids[0], ids[0] + len(ids), dtype=torch.long, device=device)
    return torch.as_tensor(ids, dtype=torch.long, device=device)


def synthetic_gpt_batch(sample_ids, sequence_length: int, vocab_size: int, device, with_labels: bool = False):
    """tokens = (id * 1103515245 + pos * 12345) mod V ; loss_mask = (id + pos) % 4 != 0.
    Returns (tokens, loss_mask, position_ids, attention_mask) -- attention_mask is None because the
    attention kernel applies the causal mask implicitly -- plus labels when `with_labels`
    (the next position's token under the same formula)."""
    ids = _ids_on_device(sample_ids, device)
    rows = ids.numel()
    if ids.is_cuda:
        from ...ops import native
        tokens = torch.empty((rows, sequence_length), dtype=torch.long, device=device)
        labels = torch.empty_like(tokens) if with_labels else None
        mask = torch.empty((rows, sequence_length), dtype=torch.float32, device=device)
        native.lib().synthetic_batch(tokens, labels, mask, ids, sequence_length, vocab_size)
    else:
        pos = torch.arange(sequence_length, dtype=torch.long, device=device).unsqueeze(0)
        base = ids.unsqueeze(1) * SYNTH_MUL
        tokens = (base + pos * SYNTH_POS) % vocab_size
        labels = (base + (pos + 1) * SYNTH_POS) % vocab_size if with_labels else None
        mask = ((ids.unsqueeze(1) + pos) % 4 != 0).float()
    position_ids = torch.arange(sequence_length, dtype=torch.long, device=device).unsqueeze(0).expand(rows, -1)
    batch = (tokens, mask, position_ids, None)
    return batch + (labels,) if with_labels else batch


# ------------------------------------------------------------------------------------------
# clock
# ------------------------------------------------------------------------------------------
@dataclass
class TrainingClock:
    total_gbs: int
    global_data_cursor: int = 0
    successful_optimizer_steps: int = 0

    def __post_init__(self):
        _positive(self.total_gbs, "total_gbs")

    def after_attempt(self, update_successful: bool) -> int:
        """Advance after one iteration; returns how many samples the LR schedule should count."""
        self.global_data_cursor += self.total_gbs
        if update_successful:
            self.successful_optimizer_steps += 1
            return self.total_gbs
        return 0

    def state(self) -> Tuple[int, int]:
        return self.global_data_cursor, self.successful_optimizer_steps


def restore_training_clock(checkpoint_args, iteration) -> Tuple[int, int]:
    """(cursor, successful steps) from the arguments stored in a checkpoint; old checkpoints that
    predate the clock fall back to consumed samples and the iteration number."""
    cursor = getattr(checkpoint_args, "global_data_cursor", getattr(checkpoint_args, "consumed_train_samples", 0))
    return cursor, getattr(checkpoint_args, "successful_optimizer_steps", iteration)


def validate_training_clock_states(states) -> None:
    states = list(states)
    if not states:
        raise ValueError("training clock states must not be empty")
    if len({tuple(s) for s in states}) != 1:
        raise ValueError(f"training clock mismatch across ranks: {tuple(states)}")
