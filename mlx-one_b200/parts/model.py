"""A model built from a ``ModelSpec`` and a set of tensors."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .base import Runtime, StepContext
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from .spec import LayerCall, ModelSpec, PartSpec, TensorSpec


def _part_tensors(registry, spec: PartSpec, prefix: str) -> dict[str, TensorSpec]:
    cls = registry.get(spec.kind)
    return {prefix + spec.stored_name(local): t for local, t in cls.tensors(spec).items()}


def expected_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    """Every stored tensor of the model by full name: the weight contract."""
    out = {spec.embedding: TensorSpec((spec.vocab_size, spec.hidden_size))}
    for layer in spec.layers:
        for registry, part in ((BLOCKS, layer.block), (MIXERS, layer.mixer),
                               (NORMS, layer.mixer_norm), (FEED_FORWARDS, layer.feed_forward),
                               (NORMS, layer.feed_forward_norm)):
            out.update(_part_tensors(registry, part, layer.prefix))
    out.update(_part_tensors(NORMS, spec.final_norm, ""))
    if spec.head is not None:
        out[spec.head] = TensorSpec((spec.vocab_size, spec.hidden_size))
    return out


def cache_entries(spec: ModelSpec) -> dict[int, Any]:
    """Cache entry -> need, for every entry that a call of the order writes."""
    needs: dict[int, Any] = {}
    for index, call in enumerate(spec.order):
        entry = index if call.cache is None else call.cache
        layer = spec.layers[call.layer]
        need = MIXERS.get(layer.mixer.kind).cache_need(layer.mixer)
        if need is None:
            continue
        if call.writes_cache:
            if entry in needs and needs[entry] != need:
                raise ValueError(f"cache entry {entry} is written with two different needs")
            needs[entry] = need
    for index, call in enumerate(spec.order):
        entry = index if call.cache is None else call.cache
        layer = spec.layers[call.layer]
        need = MIXERS.get(layer.mixer.kind).cache_need(layer.mixer)
        if need is not None and not call.writes_cache:
            if entry not in needs:
                raise ValueError(f"call {index} reads cache entry {entry} that nothing writes")
            if needs[entry] != need:
                raise ValueError(f"call {index} reads cache entry {entry} of another shape")
    return needs


class Model:
    """Embedding, layers in the spec's order, final norm and output matrix.

    ``forward(ctx)`` runs the tokens of a step and returns the 32-bit residual stream with
    the last block's output still pending; ``logits(residual, delta, rows)`` norms the
    wanted rows and multiplies them with the output matrix."""

    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor],
                 runtime: Runtime) -> None:
        self.spec = spec
        self.runtime = runtime
        self.ops = runtime.ops

        def build(registry, part: PartSpec, prefix: str, **extra):
            cls = registry.get(part.kind)
            local = {name: tensors[prefix + part.stored_name(name)]
                     for name in cls.tensors(part)}
            return cls(part, local, runtime, **extra)

        self.embedding = tensors[spec.embedding].to(runtime.dtype).contiguous()
        self.layers = []
        for layer in spec.layers:
            roles = dict(
                mixer=build(MIXERS, layer.mixer, layer.prefix),
                mixer_norm=build(NORMS, layer.mixer_norm, layer.prefix),
                feed_forward=build(FEED_FORWARDS, layer.feed_forward, layer.prefix),
                feed_forward_norm=build(NORMS, layer.feed_forward_norm, layer.prefix),
            )
            self.layers.append(build(BLOCKS, layer.block, layer.prefix, **roles))
        self.final_norm = build(NORMS, spec.final_norm, "")
        self.head = (self.embedding if spec.head is None
                     else tensors[spec.head].to(runtime.dtype).contiguous())
        self.order = tuple(
            LayerCall(call.layer, index if call.cache is None else call.cache, call.writes_cache)
            for index, call in enumerate(spec.order))
        self.cache_needs = cache_entries(spec)
        # whether steps of this model may be captured as CUDA graphs: every part says so
        parts = [self.final_norm]
        for block in self.layers:
            parts += [block, block.mixer, block.mixer_norm, block.feed_forward,
                      block.feed_forward_norm]
            position = getattr(block.mixer, "position", None)
            if position is not None:
                parts.append(position)
        self.capturable = all(getattr(part, "capturable", True) for part in parts)
        # For debugging: called as observer(place, residual, delta) after the embedding
        # (place -1) and after every call of a layer (place = its number in the order); the
        # hidden state there is residual + delta. It sees the step's own tensors: copy what is
        # to be kept. Steps that are replayed from a CUDA graph do not call it.
        self.observer = None

    def forward(self, ctx: StepContext):
        residual = self.ops.embedding(ctx.token_ids, self.embedding)
        delta = None
        if self.observer is not None:
            self.observer(-1, residual, delta)
        for place, call in enumerate(self.order):
            delta = self.layers[call.layer].forward(residual, delta, ctx,
                                                    ctx.views.get(call.cache), call.writes_cache)
            if self.observer is not None:
                self.observer(place, residual, delta)
        return residual, delta

    def logits(self, residual, delta, rows: torch.Tensor | None) -> torch.Tensor:
        """32-bit logits [len(rows), vocab] at the token rows ``rows`` (int32, device); None:
        at every row, in order (a step of single tokens that all want theirs: nothing to pick)."""
        if rows is None:
            picked, picked_delta = residual, delta
        else:
            picked, picked_delta = self.ops.gather_rows(residual, delta, rows)
        # the output product may apply the norm itself where the kernels can do that
        if self.final_norm.supports_lazy:
            normed = self.final_norm.forward(picked, picked_delta, lazy=True)
        else:
            normed = self.final_norm.forward(picked, picked_delta)
        return self.ops.linear(normed, self.head, out_dtype=torch.float32)

    def weight_bytes(self) -> int:
        """Bytes of every matrix and vector a step reads once (a tied table counts once)."""
        seen, total = set(), 0
        def visit(obj):
            nonlocal total
            for value in vars(obj).values():
                if isinstance(value, torch.Tensor):
                    key = value.data_ptr()
                    if key not in seen:
                        seen.add(key)
                        total += value.numel() * value.element_size()
                elif hasattr(value, "spec") and hasattr(value, "runtime"):
                    visit(value)
        for layer in self.layers:
            visit(layer)
        visit(self.final_norm)
        if self.head.data_ptr() not in seen:
            total += self.head.numel() * self.head.element_size()
        return total
