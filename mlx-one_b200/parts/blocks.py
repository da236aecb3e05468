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

    def forward(self, residual, delta, ctx, cache, write):
        normed = self.mixer_norm.forward(residual, delta)
        if self.mixer.fuses_residual:
            mixed = self.mixer.forward(normed, ctx, cache, write, residual=residual)
        else:
            mixed = self.mixer.forward(normed, ctx, cache, write)
        normed = self.feed_forward_norm.forward(residual, mixed)
        if self.feed_forward.fuses_residual:
            return self.feed_forward.forward(normed, ctx, residual=residual)
        return self.feed_forward.forward(normed, ctx)
