"""Normalisation parts."""

from __future__ import annotations

from .base import Norm, NormedInput
from .registry import NORMS
from .spec import TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """v * rsqrt(mean(v^2) + eps) * weight over the last axis, computed in 32-bit, fused
    with the residual add that precedes it. Parameters: ``size``, ``eps``.
    Reference: nn.RMSNorm at src/mlx_one/models/language/lfm2/reference_math.py:156-157."""

    supports_lazy = True

    @classmethod
    def tensors(cls, spec):
        return {"weight": TensorSpec((spec["size"],), "norm")}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = self.vector(tensors["weight"])
        self.eps = float(spec["eps"])

    def forward(self, residual, delta, lazy=False):
        can_fuse = getattr(self.ops, "can_fuse_norm", None)
        if lazy and delta is None and can_fuse is not None and can_fuse(residual, self.runtime.dtype):
            return NormedInput(residual, self.weight, self.eps, self.runtime.dtype, self.ops)
        return self.ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.runtime.dtype)
