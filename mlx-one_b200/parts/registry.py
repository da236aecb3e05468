"""Registries of part kinds: mixers, feed-forwards, norms, position encodings, blocks.

A part is a class registered under a kind name. Every part class provides

* ``tensors(spec) -> dict[str, TensorSpec]``: its stored tensors by local name
  (classmethod; the weight contract and the random-weights mode are built from it);
* ``__init__(spec, tensors, runtime)``: ``tensors`` maps local names to device tensors,
  ``runtime`` carries the compute dtype, the device and the kernel set.

Mixers add ``cache_need(spec)`` (classmethod) and ``forward(x, ctx, cache, write)``;
feed-forwards add ``forward(x, ctx)``; norms add ``forward(residual, delta)``;
position encodings add ``rotary_table()``; blocks add ``forward(residual, delta, ctx,
cache, write)``. The signatures are written out in ``parts/base.py``.
"""

from __future__ import annotations


class PartRegistry:
    def __init__(self, role: str) -> None:
        self.role = role
        self._kinds: dict[str, type] = {}

    def register(self, kind: str, cls: type | None = None, *, replace: bool = False):
        def put(target: type) -> type:
            if kind in self._kinds and not replace:
                raise ValueError(f"{self.role} kind {kind!r} is already registered")
            self._kinds[kind] = target
            return target
        return put if cls is None else put(cls)

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str) -> type:
        try:
            return self._kinds[kind]
        except KeyError:
            known = ", ".join(sorted(self._kinds)) or "none"
            raise KeyError(f"unknown {self.role} kind {kind!r}; registered: {known}") from None

    def kinds(self) -> tuple[str, ...]:
        return tuple(sorted(self._kinds))


MIXERS = PartRegistry("mixer")
FEED_FORWARDS = PartRegistry("feed-forward")
NORMS = PartRegistry("norm")
POSITIONS = PartRegistry("position encoding")
BLOCKS = PartRegistry("block")
