"""From a model folder to a built model."""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from ..config.registry import Architecture, read_config
from ..parts.base import Runtime
from ..parts.model import Model
from ..parts.spec import ModelSpec
from ..weights.loader import load_weights

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
          "float32": torch.float32, "fp32": torch.float32}


def resolve_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {dtype}")
        return dtype
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


@dataclass
class LoadedModel:
    path: Path
    architecture: Architecture
    config: Any
    spec: ModelSpec
    model: Model


def load_model(model_dir: str | Path, dtype: str | torch.dtype = "bfloat16",
               device: str | torch.device = "cuda:0", ops: Any = None) -> LoadedModel:
    """Reads config.json, picks the architecture from its ``model_type``, binds the
    safetensors by name and builds the model. ``ops`` is the kernel set; by default the
    CUDA extension, which is compiled here if it is not built yet."""
    path = Path(model_dir)
    dtype = resolve_dtype(dtype)
    device = torch.device(device)
    architecture, config = read_config(path)
    spec = architecture.describe(config)
    if ops is None:
        from ..kernels import default_ops
        ops = default_ops(device)
    tensors = load_weights(path, spec, dtype, device)
    model = Model(spec, tensors, Runtime(dtype, device, ops))
    return LoadedModel(path, architecture, config, spec, model)


def build_model(spec: ModelSpec, tensors, dtype, device, ops=None) -> Model:
    """A model from tensors already in memory (tests, benchmarks)."""
    dtype = resolve_dtype(dtype)
    device = torch.device(device)
    if ops is None:
        from ..kernels import default_ops
        ops = default_ops(device)
    moved = {name: t.to(device) for name, t in tensors.items()}
    return Model(spec, moved, Runtime(dtype, device, ops))
