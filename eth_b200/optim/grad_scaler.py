"""Loss scalers (reference: eth/runtime/megatron/optimizer/grad_scaler.py:66-133).

Dynamic scaler: on overflow the growth tracker resets and, once `hysteresis` overflows have been
seen, the scale is multiplied by `backoff_factor` (never below `min_scale`); after
`growth_interval` consecutive clean steps it is multiplied by `growth_factor`.
"""
from __future__ import annotations

import torch


class ConstantGradScaler:
    def __init__(self, scale: float, device="cpu"):
        if scale <= 0:
            raise ValueError("loss scale must be positive")
        self._scale = torch.tensor([float(scale)], dtype=torch.float32, device=device)
        self._value = float(scale)

    @property
    def scale(self):
        return self._scale

    @property
    def inv_scale(self) -> float:
        return 1.0 / self._value

    def value(self) -> float:
        return self._value

    def update(self, found_inf: bool) -> None:
        pass

    def state_dict(self):
        return {"scale": self._value}

    def load_state_dict(self, sd):
        pass


class DynamicGradScaler(ConstantGradScaler):
    def __init__(self, initial_scale=2.0 ** 32, min_scale=1.0, growth_factor=2.0, backoff_factor=0.5,
                 growth_interval=1000, hysteresis=2, device="cpu"):
        super().__init__(initial_scale, device)
        if not (min_scale > 0 and min_scale <= initial_scale):
            raise ValueError("min_scale must be in (0, initial_scale]")
        if growth_factor <= 1.0 or not 0.0 < backoff_factor < 1.0:
            raise ValueError("growth_factor must be > 1 and backoff_factor in (0, 1)")
        if growth_interval <= 0 or hysteresis <= 0:
            raise ValueError("growth_interval and hysteresis must be positive")
        self.min_scale, self.growth_factor, self.backoff_factor = float(min_scale), growth_factor, backoff_factor
        self.growth_interval, self.hysteresis = growth_interval, hysteresis
        self._growth_tracker = 0
        self._hysteresis_tracker = hysteresis

    def _set(self, v: float):
        self._value = v
        self._scale.fill_(v)

    def update(self, found_inf: bool) -> None:
        if found_inf:
            self._growth_tracker = 0
            self._hysteresis_tracker -= 1
            if self._hysteresis_tracker <= 0:
                self._set(max(self._value * self.backoff_factor, self.min_scale))
        else:
            self._growth_tracker += 1
            if self._growth_tracker == self.growth_interval:
                self._growth_tracker = 0
                self._hysteresis_tracker = self.hysteresis
                self._set(self._value * self.growth_factor)

    def state_dict(self):
        return {"scale": self._value, "growth_tracker": self._growth_tracker,
                "hysteresis_tracker": self._hysteresis_tracker}

    def load_state_dict(self, sd):
        self._set(float(sd["scale"]))
        self._growth_tracker = sd["growth_tracker"]
        self._hysteresis_tracker = sd["hysteresis_tracker"]
