"""Loss scalers (reference: megatron/core/optimizer/grad_scaler.py:38-142)."""
from __future__ import annotations


class ConstantGradScaler:
    def __init__(self, scale: float):
        if scale <= 0:
            raise ValueError("loss scale must be positive")
        self.scale = float(scale)

    def update(self, found_inf: bool) -> None:
        pass

    def state_dict(self):
        return {"scale": self.scale}

    def load_state_dict(self, sd):
        self.scale = sd["scale"]


class DynamicGradScaler:
    """Back off by ``backoff_factor`` after ``hysteresis`` overflowing steps; grow by
    ``growth_factor`` after ``growth_interval`` clean steps in a row."""

    def __init__(self, initial_scale, min_scale, growth_factor, backoff_factor, growth_interval, hysteresis):
        if not (initial_scale > 0 and min_scale > 0 and min_scale <= initial_scale):
            raise ValueError("bad loss-scale bounds")
        if not (growth_factor > 1.0 and 0.0 < backoff_factor < 1.0 and growth_interval > 0 and hysteresis > 0):
            raise ValueError("bad loss-scale dynamics")
        self.scale = float(initial_scale)
        self.min_scale = float(min_scale)
        self.growth_factor, self.backoff_factor = growth_factor, backoff_factor
        self.growth_interval, self.hysteresis = growth_interval, hysteresis
        self._growth_tracker = 0
        self._hysteresis_tracker = hysteresis

    def update(self, found_inf: bool) -> None:
        if found_inf:
            self._growth_tracker = 0
            self._hysteresis_tracker -= 1
            if self._hysteresis_tracker <= 0:
                self.scale = max(self.scale * self.backoff_factor, self.min_scale)
        else:
            self._growth_tracker += 1
            if self._growth_tracker == self.growth_interval:
                self._growth_tracker = 0
                self._hysteresis_tracker = self.hysteresis
                self.scale *= self.growth_factor

    def state_dict(self):
        return {"scale": self.scale, "growth_tracker": self._growth_tracker,
                "hysteresis_tracker": self._hysteresis_tracker}

    def load_state_dict(self, sd):
        self.scale = sd["scale"]
        self._growth_tracker = sd["growth_tracker"]
        self._hysteresis_tracker = sd["hysteresis_tracker"]
