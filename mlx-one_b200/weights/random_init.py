"""Random weights from a configuration and a seed, written as a model folder.

Every tensor is drawn in 32-bit on the host from a generator seeded by (seed, tensor
name), so the same folder comes out on every machine and for every order of tensors:
matrices, tables, convolution kernels and biases ~ N(0, std); norm weights ~ 1 + N(0, 0.1).
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any, Mapping

import torch

from ..config.registry import get_architecture
from ..parts.model import expected_tensors
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int.from_bytes(digest[:8], "little") >> 1)
    return generator


def random_tensors(spec, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu"):
    """name -> tensor. On the host (the default) the numbers are the documented ones; on
    another device they are drawn there, which is faster for large models and gives
    other numbers of the same distribution."""
    out = {}
    device = torch.device(device)
    for name, want in expected_tensors(spec).items():
        if device.type == "cpu":
            generator = _generator(seed, name)
        else:
            generator = torch.Generator(device=device)
            generator.manual_seed(_generator(seed, name).initial_seed())
        values = torch.randn(want.shape, generator=generator, dtype=torch.float32,
                             device=device)
        if want.init == "norm":
            values = 1.0 + 0.1 * values
        else:
            values = spec.init_std * values
        out[name] = values.to(dtype)
    return out


def write_random_model(folder: str | Path, config: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> Path:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` (the architecture's
    config.json keys, ``model_type`` included) and returns the folder."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    entry = get_architecture(config["model_type"])
    typed = entry.config_class.from_dict(config)
    spec = entry.describe(typed)
    write_safetensors(folder / "model.safetensors", random_tensors(spec, seed, dtype),
                      {"format": "pt", "seed": str(seed)})
    (folder / "config.json").write_text(json.dumps(typed.to_dict(), indent=2, sort_keys=True))
    return folder
