"""Token selection on the device for a batch of requests with their own options."""

from __future__ import annotations

from typing import Sequence

import torch

from .options import TextGenerationOptions


class Sampler:
    """Greedy where temperature is 0, else temperature / top-k / top-p sampling with a
    random number that depends only on the request's seed and on how many tokens it has
    drawn, so a request's tokens do not depend on what else is in the batch."""

    def __init__(self, ops, device) -> None:
        self.ops = ops
        self.device = torch.device(device)

    def select(self, logits: torch.Tensor, options: Sequence[TextGenerationOptions],
               steps: Sequence[int]) -> torch.Tensor:
        """logits float32 [rows, vocab] on the device -> int32 [rows] on the device."""
        if all(o.temperature == 0 for o in options):
            return self.ops.argmax(logits)
        host = torch.tensor(
            [[o.temperature, o.top_p, float(o.top_k or 0), 0.0] for o in options],
            dtype=torch.float32)
        seeds = torch.tensor([o.seed for o in options], dtype=torch.int64)
        counters = torch.tensor(list(steps), dtype=torch.int32)
        params = host.to(self.device)
        tokens, _ = self.ops.sample(
            logits, params[:, 0].contiguous(), params[:, 2].to(torch.int32).contiguous(),
            params[:, 1].contiguous(), seeds.to(self.device), counters.to(self.device))
        return tokens
