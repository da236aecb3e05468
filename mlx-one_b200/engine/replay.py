"""Replay of given token ids through the engine's own step function."""

from __future__ import annotations

from typing import Any, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from .loading import load_model
from .runner import Runner, StepEntry


class Replay:
    """A model, a cache sized for ``max_tokens`` tokens and the step function. Requests are
    opened when their first tokens arrive and closed when a step names them in ``end``."""

    def __init__(self, model_dir, *, dtype="bfloat16", max_tokens: int, page_size: int = 16,
                 device="cuda:0", max_requests: int = 64, ops: Any = None) -> None:
        if max_tokens < 1:
            raise ValueError("--max-tokens must be positive")
        if page_size < 1 or 64 % page_size:
            raise ValueError("the page size must divide 64")
        self.loaded = load_model(model_dir, dtype, device, ops)
        model = self.loaded.model
        capacity = -(-max_tokens // 64) * 64
        self.cache = CacheManager(model.cache_needs, page_size=page_size,
                                  capacity_tokens=capacity, max_requests=max_requests,
                                  dtype=model.runtime.dtype, device=model.runtime.device)
        self.runner = Runner(model, self.cache)

    def run(self, entries: Sequence[dict], end: Sequence[Any] = ()) -> np.ndarray | None:
        """One step. Returns float32 [wanted, vocab] or None if nothing was wanted."""
        batch = []
        for item in entries:
            if item["id"] not in self.cache:
                self.cache.open(item["id"])
            batch.append(StepEntry(item["id"], item["tokens"], item.get("want", ())))
        logits = self.runner.step(batch) if batch else None
        for request_id in end:
            if request_id in self.cache:
                self.cache.close(request_id)
        result = None
        if logits is not None:
            result = logits.to("cpu", torch.float32).numpy()
        self.runner.ops.check_errors()
        return result
