from . import blocks, feed_forwards, mixers, norms, positions  # register the built-in kinds
from .base import (Block, FeedForward, FixedState, Mixer, Norm, NormedInput, PagedKeyValues, PagedView,
                   Part, PositionEncoding, Runtime, StateView, StepContext)
from .model import Model, cache_entries, expected_tensors
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec, TensorSpec

__all__ = ["Block", "FeedForward", "FixedState", "Mixer", "Norm", "NormedInput", "PagedKeyValues",
           "PagedView", "Part", "PositionEncoding", "Runtime", "StateView", "StepContext",
           "Model", "cache_entries", "expected_tensors", "BLOCKS", "FEED_FORWARDS", "MIXERS",
           "NORMS", "POSITIONS", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec",
           "TensorSpec"]
