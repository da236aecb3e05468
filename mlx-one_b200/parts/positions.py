"""Position encodings."""

from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import POSITIONS


@POSITIONS.register("rope")
class RotaryEncoding(PositionEncoding):
    """Non-interleaved rotary encoding: dimension j of the first half pairs with j of the
    second half; inv_freq_j = theta^(-j / (rotary_dim / 2)), angle = position * inv_freq,
    all in 32-bit. Parameters: ``theta``, ``rotary_dim`` (even, at most the head size).
    Reference: src/mlx_one/models/shared/transformer.py:50-51, 67-72, 88-90."""

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError("rotary_dim must be positive and even")
        half = self.rotary_dim // 2
        inv_freq = torch.pow(torch.tensor(float(spec["theta"]), dtype=torch.float32),
                             -torch.arange(half, dtype=torch.float32) / half)
        self.inv_freq = inv_freq.to(runtime.device)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim


@POSITIONS.register("none")
class NoPositionEncoding(PositionEncoding):
    """No rotation: order is known to the model only through causality."""

    def rotary_table(self):
        return None
