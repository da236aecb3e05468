"""Feed-forward parts."""

from __future__ import annotations

import torch

from .base import FeedForward
from .registry import FEED_FORWARDS
from .spec import TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """w2(silu(w1 x) * w3 x), no biases. Parameters: ``hidden``, ``width``. The gate and
    up matrices are stacked at load time so that one matrix product feeds the gate kernel.
    Reference: src/mlx_one/models/language/lfm2/reference_math.py:114-135."""

    @classmethod
    def tensors(cls, spec):
        hidden, width = spec["hidden"], spec["width"]
        return {
            "w1.weight": TensorSpec((width, hidden)),
            "w3.weight": TensorSpec((width, hidden)),
            "w2.weight": TensorSpec((hidden, width)),
        }

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.width = spec["width"]
        self.gate_up = self.matrix(torch.cat([tensors["w1.weight"], tensors["w3.weight"]], dim=0))
        self.down = self.matrix(tensors["w2.weight"])

    fuses_residual = True
    accepts_normed_input = True

    def forward(self, x, ctx, residual=None):
        gated = self.ops.linear_swiglu(x, self.gate_up)
        if residual is None:
            return self.ops.linear(gated, self.down)
        return self.ops.linear_add(gated, self.down, None, residual)
