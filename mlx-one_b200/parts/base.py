"""Interfaces of the parts and of what they are given at run time."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

import torch

from .spec import PartSpec, TensorSpec


# ----------------------------------------------------------------------- cache needs


@dataclass(frozen=True)
class PagedKeyValues:
    """A mixer that keeps a key and a value vector per token and per key head. Layers
    whose need is equal share pages and a block table. ``window``: only the last
    ``window`` positions are ever read again, so earlier pages may be given back."""

    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class FixedState:
    """A mixer with per-request state of fixed size (``shape`` per cache entry), kept in
    a slot. The slot is zero when a request gets it."""

    shape: tuple[int, ...]
    dtype: str = "compute"          # "compute" = the engine's dtype, or "float32"


# ----------------------------------------------------------------------- run time


@dataclass
class Runtime:
    """What a part needs besides its tensors: compute dtype, device and kernels."""

    dtype: torch.dtype
    device: torch.device
    ops: Any


@dataclass
class PagedView:
    """One cache entry of a paged group as a step sees it. ``kv`` is
    [2, pages, kv_heads, page_size, head_dim]; ``block_table`` is int32 [requests, width]
    with -1 where a page was given back."""

    kv: torch.Tensor
    block_table: torch.Tensor
    page_size: int
    need: PagedKeyValues


@dataclass
class StateView:
    """One cache entry of a fixed-state group: ``state`` is [slots, *shape] and
    ``slots`` int32 [requests] names each request's slot."""

    state: torch.Tensor
    slots: torch.Tensor
    need: FixedState


@dataclass
class StepContext:
    """The ragged batch of one step. All tensors are int32 on the device.

    ``token_ids``/``positions``/``token_request`` have one entry per token; tokens of a
    request are consecutive and in order. ``request_start`` [requests + 1] are offsets
    into the tokens; ``history`` [requests] is each request's token count before this
    step (the position of its first token here).

    Host values and CUDA graphs. A step whose shape (requests, tokens, table widths, wanted
    rows) comes back may be captured as a CUDA graph and replayed with other contents: other
    token ids, positions, tables, and another split of the tokens between the requests. What a
    part reads on the host while it is captured is frozen into the graph. Therefore, in a step
    that may be captured (``replayable`` True), ``max_portion`` and ``max_context`` are upper
    bounds that hold for every step of that shape (``max_portion`` is 1 exactly when every
    request brings one token), and ``host`` refuses to be read. A part that needs the step's
    own host values (or synchronises, or runs host code per request) sets ``capturable =
    False`` on its class; a model with such a part is never captured."""

    tokens: int
    requests: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_request: torch.Tensor
    request_start: torch.Tensor
    history: torch.Tensor
    max_portion: int                  # most tokens any request brings (host; see above)
    max_context: int                  # largest history + portion (host; see above)
    views: Mapping[int, Any] = field(default_factory=dict)   # cache entry -> view
    # host copies of ``history`` and ``request_start`` (lists), for parts that are not capturable
    host: Mapping[str, Any] = field(default_factory=dict)
    replayable: bool = False
    # The first ``leading_single`` requests bring exactly one token each (token i is request
    # i's): the decodes at the head of a step. A host value that is part of a captured step's
    # shape, so it holds for every replay. A mixer may give these tokens to a kernel made for
    # single tokens and the rest to another.
    leading_single: int = 0


class NoHostValues(Mapping):
    """``StepContext.host`` of a step that may be replayed from a CUDA graph: reading it would
    freeze one step's values into the graph, so it raises instead."""

    def __getitem__(self, key):
        raise RuntimeError(
            f"StepContext.host[{key!r}] was read in a step that may be captured as a CUDA graph; "
            "a part that needs host values sets `capturable = False` on its class")

    def __iter__(self):
        return iter(())

    def __len__(self):
        return 0


class NormedInput:
    """The output of a norm that has not been computed yet: the 32-bit rows, the norm's weight
    and eps. A kernel set that can apply the norm while it loads its input takes this as the
    input of ``linear`` / ``linear_swiglu``; ``materialize()`` computes it the ordinary way.
    Only parts that declare ``accepts_normed_input`` are ever given one."""

    def __init__(self, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                 dtype: torch.dtype, ops: Any) -> None:
        self.residual, self.weight, self.eps, self.dtype, self.ops = residual, weight, eps, dtype, ops
        self.shape = residual.shape

    def materialize(self) -> torch.Tensor:
        return self.ops.add_rmsnorm(self.residual, None, self.weight, self.eps, self.dtype)


# ----------------------------------------------------------------------- part bases


class Part:
    """Common construction: checks that the given tensors match ``tensors(spec)``."""

    # False: this part's forward cannot be recorded into a CUDA graph and replayed with other
    # contents (it reads ``StepContext.host``, copies to the host, or loops over requests in
    # Python). A model that holds such a part runs every step eagerly.
    capturable = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor],
                 runtime: Runtime) -> None:
        self.spec = spec
        self.runtime = runtime
        self.ops = runtime.ops
        expected = self.tensors(spec)
        for name, want in expected.items():
            if name not in tensors:
                raise KeyError(f"{type(self).__name__}: tensor {name!r} was not given")
            if tuple(tensors[name].shape) != tuple(want.shape):
                raise ValueError(f"{type(self).__name__}: {name} has shape "
                                 f"{tuple(tensors[name].shape)}, expected {want.shape}")

    @classmethod
    def tensors(cls, spec: PartSpec) -> dict[str, TensorSpec]:
        return {}

    def matrix(self, tensor: torch.Tensor) -> torch.Tensor:
        """A matrix operand in the compute dtype."""
        return tensor.to(self.runtime.dtype).contiguous()

    def vector(self, tensor: torch.Tensor) -> torch.Tensor:
        """A small per-channel vector, read by kernels in 32-bit (exact from bfloat16)."""
        return tensor.to(torch.float32).contiguous()


class Mixer(Part):
    # True: forward takes ``residual=`` and may add its output there itself, returning None
    fuses_residual = False
    # True: the input is used only as the input of ops.linear / ops.linear_swiglu, so it may be
    # a NormedInput (the norm then happens inside that product where the kernels can do it)
    accepts_normed_input = False

    @classmethod
    def cache_need(cls, spec: PartSpec):
        """``PagedKeyValues``, ``FixedState`` or None."""
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Any, write: bool):
        """x: normed input [tokens, hidden] in the compute dtype. Returns the mixer's
        output [tokens, hidden] in the compute dtype (the block adds it to the
        residual). ``write``: append this step's tokens to ``cache``."""
        raise NotImplementedError


class FeedForward(Part):
    fuses_residual = False      # as for mixers
    accepts_normed_input = False

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    # True: forward takes ``lazy=`` (see below); a norm that leaves it False is always computed
    supports_lazy = False

    def forward(self, residual: torch.Tensor, delta: torch.Tensor | None,
                lazy: bool = False) -> torch.Tensor:
        """Adds ``delta`` (compute dtype, or None) into the 32-bit ``residual`` in place
        and returns the normed residual in the compute dtype. With ``lazy`` a norm may return
        a ``NormedInput`` instead, for a consumer that ``accepts_normed_input``."""
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_table(self) -> tuple[torch.Tensor, int] | None:
        """(inverse frequencies [rotary_dim / 2] float32, rotary_dim) for encodings that
        rotate queries and keys by position * frequency; None for no rotation."""
        return None


class Block(Part):
    """Arranges a layer's parts. Gets the built parts by role."""

    def __init__(self, spec, tensors, runtime, *, mixer, mixer_norm, feed_forward,
                 feed_forward_norm) -> None:
        super().__init__(spec, tensors, runtime)
        self.mixer = mixer
        self.mixer_norm = mixer_norm
        self.feed_forward = feed_forward
        self.feed_forward_norm = feed_forward_norm

    def forward(self, residual: torch.Tensor, delta: torch.Tensor | None, ctx: StepContext,
                cache: Any, write: bool) -> torch.Tensor | None:
        """``residual`` is the 32-bit stream [tokens, hidden], updated in place; ``delta``
        is an output of the previous block that is still to be added (or None). Returns
        this block's pending output in the same way."""
        raise NotImplementedError
