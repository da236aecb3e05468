"""The step function: one ragged batch of (request, its next tokens) through the model.

A step takes, for every request in it, the tokens that come next (a portion of a prompt, or
one decoded token), runs exactly these tokens as one batch against what earlier steps left
in the cache, appends their keys, values and state, and returns the 32-bit logits at the
places asked for. A decoded token is simply a portion of length one, so prompts and decodes
mix freely. The reference runs one phase per batch and pads to the widest row
(src/mlx_one/engine/hybrid.py:115-252); here nothing is padded.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

import torch

from ..cache.manager import CacheManager
from ..parts.base import StepContext
from ..parts.model import Model


@dataclass
class StepEntry:
    """One request's share of a step. ``want``: places among ``tokens`` whose logits are
    returned (in this order)."""

    request_id: Any
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


def _align(value: int, to: int = 4) -> int:
    return -(-value // to) * to


class Runner:
    def __init__(self, model: Model, cache: CacheManager) -> None:
        self.model = model
        self.cache = cache
        self.ops = model.ops
        self.device = model.runtime.device
        self._staging: list[torch.Tensor | None] = [None, None]
        self._events: list[Any] = [None, None]
        self._device_buffer: torch.Tensor | None = None
        self._turn = 0
        self.steps = 0
        self.last_shape = (0, 0)

    # ------------------------------------------------------------------ staging

    def _host_buffer(self, size: int) -> torch.Tensor:
        """A host int32 buffer of at least ``size`` entries whose last copy has landed."""
        self._turn ^= 1
        turn = self._turn
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        buffer = self._staging[turn]
        if buffer is None or buffer.numel() < size:
            capacity = max(1024, 1 << (size - 1).bit_length())
            buffer = torch.empty(capacity, dtype=torch.int32,
                                 pin_memory=self.device.type == "cuda")
            self._staging[turn] = buffer
        if self._device_buffer is None or self._device_buffer.numel() < buffer.numel():
            self._device_buffer = torch.empty(buffer.numel(), dtype=torch.int32,
                                              device=self.device)
        return buffer

    # ------------------------------------------------------------------ the step

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor | None:
        """Runs the entries as one batch. Returns float32 logits [wanted, vocab] on the
        device in the order of the entries and of their ``want``, or None if nothing is
        wanted. Raises before touching any state if the batch is malformed or pages run
        out (``CacheCapacityError``)."""
        if not entries:
            return None
        vocab = self.model.spec.vocab_size
        seen = set()
        for entry in entries:
            if entry.request_id in seen:
                raise ValueError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            if len(entry.tokens) < 1:
                raise ValueError(f"request {entry.request_id!r} brings no tokens")
            for token in entry.tokens:
                if not 0 <= int(token) < vocab:
                    raise ValueError(f"token {token} is outside the vocabulary of {vocab}")
            for place in entry.want:
                if not 0 <= int(place) < len(entry.tokens):
                    raise ValueError(f"wanted place {place} is outside the request's tokens")
            limit = self.model.spec.max_positions
            held = self.cache.get(entry.request_id).length
            if held + len(entry.tokens) > limit:
                raise ValueError(f"request {entry.request_id!r} would pass the model's "
                                 f"{limit} positions")
        for entry in entries:
            self.cache.grow(entry.request_id, len(entry.tokens))

        requests = len(entries)
        tokens = sum(len(e.tokens) for e in entries)
        wanted = sum(len(e.want) for e in entries)
        caches = [self.cache.get(e.request_id) for e in entries]
        paged, states = self.cache.paged, self.cache.states
        widths = [_align(max(max(len(c.tables[g]) for c in caches), 1), 8)
                  for g in range(len(paged))]

        # one packed int32 buffer: five per-token and per-request lists, block tables, slots
        offsets, cursor = {}, 0
        def region(name: str, size: int) -> None:
            nonlocal cursor
            offsets[name] = (cursor, size)
            cursor = _align(cursor + size)
        region("token_ids", tokens)
        region("positions", tokens)
        region("token_request", tokens)
        region("request_start", requests + 1)
        region("history", requests)
        region("rows", max(wanted, 1))
        for g in range(len(paged)):
            region(f"table{g}", requests * widths[g])
        for g in range(len(states)):
            region(f"slots{g}", requests)
        host = self._host_buffer(cursor)
        data = host.numpy()

        def put(name: str, values) -> None:
            start, size = offsets[name]
            data[start:start + size] = values

        token_ids, positions, token_request, starts, history, rows = [], [], [], [0], [], []
        for r, (entry, cache) in enumerate(zip(entries, caches)):
            n = len(entry.tokens)
            first = len(token_ids)
            token_ids.extend(int(t) for t in entry.tokens)
            positions.extend(range(cache.length, cache.length + n))
            token_request.extend([r] * n)
            starts.append(first + n)
            history.append(cache.length)
            rows.extend(first + int(place) for place in entry.want)
        put("token_ids", token_ids)
        put("positions", positions)
        put("token_request", token_request)
        put("request_start", starts)
        put("history", history)
        put("rows", rows if rows else [0])
        for g in range(len(paged)):
            start, size = offsets[f"table{g}"]
            table = data[start:start + size].reshape(requests, widths[g])
            table[:] = -1
            for r, cache in enumerate(caches):
                table[r, :len(cache.tables[g])] = cache.tables[g]
        for g in range(len(states)):
            put(f"slots{g}", [c.slots[g] for c in caches])

        device = self._device_buffer
        device[:cursor].copy_(host[:cursor], non_blocking=True)
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
            self._events[self._turn] = event

        def on_device(name: str) -> torch.Tensor:
            start, size = offsets[name]
            return device[start:start + size]

        tables = [on_device(f"table{g}").view(requests, widths[g]) for g in range(len(paged))]
        slots = [on_device(f"slots{g}") for g in range(len(states))]
        views = {entry: self.cache.view(entry, tables, slots) for entry in self.model.cache_needs}
        ctx = StepContext(
            tokens=tokens, requests=requests, token_ids=on_device("token_ids"),
            positions=on_device("positions"), token_request=on_device("token_request"),
            request_start=on_device("request_start"), history=on_device("history"),
            max_portion=max(len(e.tokens) for e in entries),
            max_context=max(h + len(e.tokens) for h, e in zip(history, entries)),
            views=views,
            host={"history": history, "request_start": starts, "positions": positions,
                  "token_request": token_request})

        residual, delta = self.model.forward(ctx)
        logits = None
        if wanted:
            logits = self.model.logits(residual, delta, on_device("rows")[:wanted])
        for entry in entries:
            self.cache.advance(entry.request_id, len(entry.tokens))
        self.steps += 1
        self.last_shape = (requests, tokens)
        return logits
