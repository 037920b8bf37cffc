"""Learning-rate schedule counted in samples: linear warm-up, then constant / linear / cosine decay
to `min_lr` (reference: eth/runtime/megatron/learning_rates.py:58-99; the trainer advances it by
`total_gbs` per successful step, training.py:1029)."""
from __future__ import annotations

import math


class AnnealingLR:
    def __init__(self, optimizer, max_lr, min_lr, warmup_steps, decay_steps, decay_style="cosine",
                 use_checkpoint_lr_scheduler=True, override_lr_scheduler=False):
        self.optimizer = optimizer
        self.max_lr, self.min_lr = float(max_lr), float(min_lr)
        if self.min_lr < 0 or self.max_lr < self.min_lr:
            raise ValueError("need 0 <= min_lr <= max_lr")
        self.warmup_steps, self.decay_steps = warmup_steps, decay_steps
        if decay_steps <= 0 or warmup_steps >= decay_steps:
            raise ValueError("need 0 <= warmup_steps < decay_steps")
        if decay_style not in ("constant", "linear", "cosine"):
            raise ValueError(f"{decay_style} decay style is not supported")
        self.decay_style = decay_style
        self.num_steps = 0
        self.override_lr_scheduler = override_lr_scheduler
        self.use_checkpoint_lr_scheduler = use_checkpoint_lr_scheduler
        if override_lr_scheduler and use_checkpoint_lr_scheduler:
            raise ValueError("both override and use-checkpoint are set")
        self.step(0)

    def get_lr(self) -> float:
        if self.warmup_steps > 0 and self.num_steps <= self.warmup_steps:
            return self.max_lr * float(self.num_steps) / float(self.warmup_steps)
        if self.decay_style == "constant":
            return self.max_lr
        if self.num_steps > self.decay_steps:
            return self.min_lr
        ratio = float(self.num_steps - self.warmup_steps) / float(self.decay_steps - self.warmup_steps)
        delta = self.max_lr - self.min_lr
        if self.decay_style == "linear":
            coeff = 1.0 - ratio
        else:
            coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
        return self.min_lr + coeff * delta

    def step(self, increment: int) -> None:
        self.num_steps += increment
        lr = self.get_lr()
        if self.optimizer is not None:
            self.optimizer.set_lr(lr)

    def state_dict(self):
        return {"max_lr": self.max_lr, "warmup_steps": self.warmup_steps, "num_steps": self.num_steps,
                "decay_style": self.decay_style, "decay_steps": self.decay_steps, "min_lr": self.min_lr}

    def _check(self, mine, theirs, what):
        if self.override_lr_scheduler:
            return mine
        if not self.use_checkpoint_lr_scheduler and mine != theirs:
            raise ValueError(f"AnnealingLR: class input value {mine} and checkpoint value {theirs} for {what} do not match")
        return theirs

    def load_state_dict(self, sd):
        self.max_lr = self._check(self.max_lr, sd["max_lr"], "learning rate")
        self.min_lr = self._check(self.min_lr, sd["min_lr"], "minimum learning rate")
        self.warmup_steps = self._check(self.warmup_steps, sd["warmup_steps"], "warmup iterations")
        self.decay_steps = self._check(self.decay_steps, sd["decay_steps"], "total number of iterations")
        self.decay_style = self._check(self.decay_style, sd["decay_style"], "decay style")
        self.num_steps = 0
        self.step(sd["num_steps"])
