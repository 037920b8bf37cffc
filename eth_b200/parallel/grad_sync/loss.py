"""Global loss normalisation, sample ownership and the training clock.

Contract (reference: eth/runtime/megatron/grad_sync/loss.py):
  * a forward step returns `LossOutput(local_loss_sum, local_loss_weight, nominal scale)`; the value
    that is back-propagated is `local_loss_sum / nominal_global_loss_scale`, and after all
    micro-batches the gradients are multiplied by `nominal / sum_world(loss_weight)` (:33-39);
  * sample slots: pipeline offset + micro-batch prefix + dp_rank * local_mbs, from the global data
    cursor (:70-97);
  * the synthetic batch is a closed formula of (sample id, position) (:100-119);
  * the clock advances the data cursor on every attempt and the step counter only on success
    (:122-137).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch


@dataclass(frozen=True)
class LossOutput:
    local_loss_sum: object
    local_loss_weight: object
    nominal_global_loss_scale: float
    metrics: dict


def gpt_loss_output(losses, loss_mask, nominal_global_loss_scale, metrics=None) -> LossOutput:
    if nominal_global_loss_scale <= 0:
        raise ValueError("nominal_global_loss_scale must be positive")
    flat = losses.float().reshape(-1)
    mask = loss_mask.float().reshape(-1)
    if flat.numel() != mask.numel():
        raise ValueError("GPT loss and loss_mask must have the same numel")
    return LossOutput(torch.sum(flat * mask), torch.sum(mask), float(nominal_global_loss_scale),
                      {} if metrics is None else metrics)


def global_normalization_scale(nominal_global_loss_scale, global_loss_weight):
    if nominal_global_loss_scale <= 0:
        raise ValueError("nominal_global_loss_scale must be positive")
    if float(global_loss_weight.detach().item()) <= 0:
        raise ValueError("global_loss_weight must be positive")
    return nominal_global_loss_scale / global_loss_weight


def sum_loss_outputs(outputs):
    outputs = tuple(outputs)
    if not outputs:
        raise ValueError("loss_outputs must not be empty")
    return sum(o.local_loss_sum for o in outputs), sum(o.local_loss_weight for o in outputs)


def restore_training_clock(checkpoint_args, iteration):
    consumed = getattr(checkpoint_args, "consumed_train_samples", 0)
    return (getattr(checkpoint_args, "global_data_cursor", consumed),
            getattr(checkpoint_args, "successful_optimizer_steps", iteration))


def validate_training_clock_states(states) -> None:
    states = tuple(states)
    if not states:
        raise ValueError("training clock states must not be empty")
    if any(s != states[0] for s in states[1:]):
        raise ValueError(f"training clock mismatch across ranks: {states}")


def local_sample_slots(pipeline_id: int, microbatch_index: int, dp_degree: int, dp_rank: int,
                       mbs_sequences: Sequence, pipeline_sample_offsets: Sequence[int], global_data_cursor: int):
    if not 0 <= pipeline_id < len(mbs_sequences):
        raise ValueError(f"unknown pipeline_id {pipeline_id}")
    seq = mbs_sequences[pipeline_id]
    if not 0 <= microbatch_index < len(seq):
        raise ValueError(f"unknown microbatch_index {microbatch_index}")
    if dp_degree <= 0 or not 0 <= dp_rank < dp_degree:
        raise ValueError("invalid DP coordinate")
    global_mbs = seq[microbatch_index][0]
    if global_mbs % dp_degree:
        raise ValueError("global microbatch size must be divisible by DP degree")
    local = global_mbs // dp_degree
    begin = (global_data_cursor + pipeline_sample_offsets[pipeline_id]
             + sum(item[0] for item in seq[:microbatch_index]) + dp_rank * local)
    return tuple(range(begin, begin + local))


SYNTH_MUL, SYNTH_POS = 1103515245, 12345


def synthetic_gpt_batch(sample_ids, sequence_length: int, vocab_size: int, device, with_labels: bool = False):
    """tokens = (id * 1103515245 + pos * 12345) mod V ; loss_mask = (id + pos) % 4 != 0.
    Returns (tokens, loss_mask, position_ids, attention_mask) -- attention_mask is None because the
    attention kernel applies the causal mask implicitly -- plus labels when `with_labels`
    (the next position's token under the same formula)."""
    sample_ids = tuple(sample_ids) if not isinstance(sample_ids, torch.Tensor) else sample_ids
    if (not isinstance(sample_ids, torch.Tensor) and len(sample_ids) > 0
            and sample_ids[-1] - sample_ids[0] == len(sample_ids) - 1):
        # consecutive slots: build the ids on the device (a host->device copy would synchronise)
        ids = torch.arange(sample_ids[0], sample_ids[0] + len(sample_ids), dtype=torch.long, device=device)
    else:
        ids = torch.as_tensor(sample_ids, dtype=torch.long, device=device)
    n = ids.numel()
    if ids.is_cuda:
        from ...ops import native
        tokens = torch.empty((n, sequence_length), dtype=torch.long, device=device)
        labels = torch.empty_like(tokens) if with_labels else None
        mask = torch.empty((n, sequence_length), dtype=torch.float32, device=device)
        native.lib().synthetic_batch(tokens, labels, mask, ids, sequence_length, vocab_size)
    else:
        pos = torch.arange(sequence_length, dtype=torch.long, device=device)
        tokens = (ids[:, None] * SYNTH_MUL + pos[None, :] * SYNTH_POS).remainder(vocab_size)
        mask = ((ids[:, None] + pos[None, :]) % 4 != 0).float()
        labels = (ids[:, None] * SYNTH_MUL + (pos[None, :] + 1) * SYNTH_POS).remainder(vocab_size) if with_labels else None
    position_ids = torch.arange(sequence_length, dtype=torch.long, device=device)[None, :].expand(n, -1)
    if with_labels:
        return tokens, mask, position_ids, None, labels
    return tokens, mask, position_ids, None


@dataclass
class TrainingClock:
    total_gbs: int
    global_data_cursor: int = 0
    successful_optimizer_steps: int = 0

    def __post_init__(self):
        if self.total_gbs <= 0:
            raise ValueError("total_gbs must be positive")

    def after_attempt(self, update_successful: bool) -> int:
        self.global_data_cursor += self.total_gbs
        if not update_successful:
            return 0
        self.successful_optimizer_steps += 1
        return self.total_gbs
