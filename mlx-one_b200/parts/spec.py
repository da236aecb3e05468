"""Plain data that describes a model: which parts, with which constants, in which order.

A ``ModelSpec`` is what an architecture's ``describe(config)`` returns. Nothing in it
is executable: parts are named by kind and looked up in the part registries when the
model is built, so a model may use a different mixer or feed-forward in every layer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind, its sizes and constants, and the prefix (relative
    to the layer's prefix) under which its tensors are stored. ``names`` maps the part's
    own tensor names to other stored names where an architecture calls them differently."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""
    names: Mapping[str, str] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def stored_name(self, local: str) -> str:
        return self.prefix + self.names.get(local, local)


@dataclass(frozen=True)
class TensorSpec:
    """Shape of a stored tensor and how the random-weights mode fills it:
    ``normal`` ~ N(0, std), ``norm`` ~ 1 + N(0, 0.1), ``bias`` ~ N(0, std)."""

    shape: tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement and the parts it arranges, by role."""

    prefix: str
    block: PartSpec
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class LayerCall:
    """One entry of the execution order. ``layer`` indexes ``ModelSpec.layers`` and may
    appear more than once. ``cache`` names the cache entry that the call's mixer uses;
    by default every call has an entry of its own (its index in the order). A call with
    ``writes_cache=False`` reads an entry that an earlier call of the step has written."""

    layer: int
    cache: int | None = None
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: str                          # stored name of the [vocab, hidden] table
    layers: tuple[LayerSpec, ...]
    order: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: str | None                        # stored name of the output matrix; None = tied
    max_positions: int
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    init_std: float = 0.02
    # (stored name, shape) -> (name, squeeze axis or None), or None to drop the tensor
    rename: Callable[[str, tuple[int, ...]], tuple[str, int | None] | None] | None = None
