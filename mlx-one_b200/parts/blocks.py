"""Arrangements of a layer's parts."""

from __future__ import annotations

from .base import Block
from .registry import BLOCKS


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """h = x + mixer(norm(x)); out = h + feed_forward(norm(h)). Each residual add is fused
    with the norm that follows it, so the block returns its last output unadded; a part that
    ``fuses_residual`` may instead add its output into the stream itself and return None.
    Reference: src/mlx_one/models/language/lfm2/reference_math.py:160-179."""

    @staticmethod
    def _norm(norm, residual, delta, consumer):
        if consumer.accepts_normed_input and norm.supports_lazy:
            return norm.forward(residual, delta, lazy=True)
        return norm.forward(residual, delta)

    def forward(self, residual, delta, ctx, cache, write):
        normed = self._norm(self.mixer_norm, residual, delta, self.mixer)
        if self.mixer.fuses_residual:
            mixed = self.mixer.forward(normed, ctx, cache, write, residual=residual)
        else:
            mixed = self.mixer.forward(normed, ctx, cache, write)
        normed = self._norm(self.feed_forward_norm, residual, mixed, self.feed_forward)
        if self.feed_forward.fuses_residual:
            return self.feed_forward.forward(normed, ctx, residual=residual)
        return self.feed_forward.forward(normed, ctx)
