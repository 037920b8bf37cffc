"""Learning-rate schedule counted in samples.

The schedule itself is a pure function of the sample count (`Schedule.at`): a linear ramp from 0
to the peak over the warm-up, then the peak (constant), a straight line or half a cosine down to
the floor at `decay_steps`, and the floor from there on. `AnnealingLR` is the stateful wrapper the
trainer holds: it counts samples (the trainer advances it by the global batch size per successful
step), pushes the value into the optimizer, and round-trips through checkpoints with the
reference's keys and override rules (reference: eth/runtime/megatron/learning_rates.py:58-99 the
formula, :101-164 state and the checkpoint policy; training.py:1029 the advance).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

SHAPES = {
    "constant": lambda progress: 1.0,
    "linear": lambda progress: 1.0 - progress,
    "cosine": lambda progress: 0.5 * (1.0 + math.cos(math.pi * progress)),
}


@dataclass
class Schedule:
    peak: float
    floor: float
    warmup_steps: int
    decay_steps: int
    style: str = "cosine"

    def __post_init__(self):
        if self.floor < 0 or self.peak < self.floor:
            raise ValueError("need 0 <= min_lr <= max_lr")
        if self.decay_steps <= 0 or self.warmup_steps >= self.decay_steps:
            raise ValueError("need 0 <= warmup_steps < decay_steps")
        if self.style not in SHAPES:
            raise ValueError(f"{self.style} decay style is not supported")

    def at(self, count: int) -> float:
        if 0 < self.warmup_steps and count <= self.warmup_steps:
            return self.peak * count / self.warmup_steps
        if self.style == "constant":
            return self.peak
        if count > self.decay_steps:
            return self.floor
        progress = (count - self.warmup_steps) / (self.decay_steps - self.warmup_steps)
        return self.floor + SHAPES[self.style](progress) * (self.peak - self.floor)


# checkpoint key -> (Schedule field, what to call it in a mismatch message)
_PERSISTED = (("max_lr", "peak", "learning rate"), ("min_lr", "floor", "minimum learning rate"),
              ("warmup_steps", "warmup_steps", "warmup iterations"),
              ("decay_steps", "decay_steps", "total number of iterations"), ("decay_style", "style", "decay style"))


class AnnealingLR:
    def __init__(self, optimizer, max_lr, min_lr, warmup_steps, decay_steps, decay_style="cosine",
                 use_checkpoint_lr_scheduler=True, override_lr_scheduler=False):
        if override_lr_scheduler and use_checkpoint_lr_scheduler:
            raise ValueError("both override and use-checkpoint are set")
        self.optimizer = optimizer
        self.schedule = Schedule(float(max_lr), float(min_lr), warmup_steps, decay_steps, decay_style)
        self.use_checkpoint_lr_scheduler, self.override_lr_scheduler = use_checkpoint_lr_scheduler, override_lr_scheduler
        self.num_steps = 0
        self.step(0)

    # the fields other modules read
    max_lr = property(lambda self: self.schedule.peak)
    min_lr = property(lambda self: self.schedule.floor)
    warmup_steps = property(lambda self: self.schedule.warmup_steps)
    decay_steps = property(lambda self: self.schedule.decay_steps)
    decay_style = property(lambda self: self.schedule.style)

    def get_lr(self) -> float:
        return self.schedule.at(self.num_steps)

    def step(self, increment: int) -> None:
        self.num_steps += increment
        if self.optimizer is not None:
            self.optimizer.set_lr(self.get_lr())

    def state_dict(self):
        state = {key: getattr(self.schedule, field) for key, field, _ in _PERSISTED}
        state["num_steps"] = self.num_steps
        return state

    def load_state_dict(self, sd):
        """Checkpoint values win unless `override_lr_scheduler`; with neither flag set, a value that
        differs from the command line is an error."""
        for key, field, what in _PERSISTED:
            mine, theirs = getattr(self.schedule, field), sd[key]
            if self.override_lr_scheduler:
                continue
            if not self.use_checkpoint_lr_scheduler and mine != theirs:
                raise ValueError(f"AnnealingLR: class input value {mine} and checkpoint value {theirs} for {what} "
                                 "do not match")
            setattr(self.schedule, field, theirs)
        self.num_steps = 0
        self.step(sd["num_steps"])
