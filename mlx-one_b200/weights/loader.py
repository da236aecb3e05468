"""Binding stored tensors to a model by name.

Tensors are renamed as the architecture asks, checked against the model's expected names
and shapes, and copied to the device. All problems are reported in one error that lists
missing tensors, unexpected tensors and wrong shapes, as the reference's contract does
(src/mlx_one/core/weights.py:20-46).

dtypes: in the bfloat16 engine, 16-bit floating tensors are kept in bfloat16 and tensors
stored in 32-bit stay in 32-bit (a part casts a matrix operand when it is built); in the
float32 engine every floating tensor is promoted to float32. Integer tensors become int32.
"""

from __future__ import annotations

from pathlib import Path
from typing import Mapping

import torch

from ..parts.model import expected_tensors
from ..parts.spec import ModelSpec
from .safetensors_io import SafetensorsError, SafetensorsFile, checkpoint_files, checkpoint_index


class WeightError(ValueError):
    """Stored tensors do not match the model. ``missing``, ``unexpected`` and
    ``mismatched`` hold the names."""

    def __init__(self, missing, unexpected, mismatched, duplicates=()):
        self.missing = tuple(missing)
        self.unexpected = tuple(unexpected)
        self.mismatched = tuple(mismatched)
        self.duplicates = tuple(duplicates)
        problems = []
        if self.missing:
            problems.append("missing tensors: " + ", ".join(self.missing))
        if self.unexpected:
            problems.append("unexpected tensors: " + ", ".join(self.unexpected))
        if self.mismatched:
            problems.append("wrong shapes: " + ", ".join(
                f"{name} is {got} but should be {want}" for name, got, want in self.mismatched))
        if self.duplicates:
            problems.append("tensors stored twice: " + ", ".join(self.duplicates))
        super().__init__("; ".join(problems))


def _kept_dtype(stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32 or stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_names(spec: ModelSpec, stored: Mapping[str, tuple[int, ...]]):
    """Applies the architecture's renames to ``stored`` (name -> shape) and compares with
    the model's expectation. Returns {engine name: (stored name, squeeze axis)}; raises
    ``WeightError`` listing everything that is wrong."""
    expected = expected_tensors(spec)
    bound: dict[str, tuple[str, int | None]] = {}
    shapes: dict[str, tuple[int, ...]] = {}
    duplicates = []
    for name, shape in stored.items():
        renamed = (name, None) if spec.rename is None else spec.rename(name, tuple(shape))
        if renamed is None:
            continue
        new_name, axis = renamed
        if new_name in bound:
            duplicates.append(new_name)
            continue
        shape = tuple(shape)
        if axis is not None:
            shape = shape[:axis] + shape[axis + 1:]
        bound[new_name] = (name, axis)
        shapes[new_name] = shape
    missing = sorted(set(expected) - set(bound))
    unexpected = sorted(set(bound) - set(expected))
    mismatched = sorted((name, shapes[name], tuple(expected[name].shape))
                        for name in set(bound) & set(expected)
                        if shapes[name] != tuple(expected[name].shape))
    if missing or unexpected or mismatched or duplicates:
        raise WeightError(missing, unexpected, mismatched, sorted(duplicates))
    return bound


def load_weights(model_dir: str | Path, spec: ModelSpec, dtype: torch.dtype,
                 device: torch.device | str) -> dict[str, torch.Tensor]:
    files = [SafetensorsFile(path) for path in checkpoint_files(model_dir)]
    try:
        stored: dict[str, tuple[int, ...]] = {}
        where: dict[str, SafetensorsFile] = {}
        twice = []
        for handle in files:
            for name, (_, shape) in handle.entries.items():
                if name in stored:
                    twice.append(name)
                stored[name] = shape
                where[name] = handle
        if twice:
            raise WeightError((), (), (), sorted(twice))
        weight_map = checkpoint_index(model_dir)
        if weight_map is not None:
            # the index and the shards must say the same (src/mlx_one/text/loading.py:547-554)
            astray = sorted(name for name, handle in where.items()
                            if weight_map.get(name) != handle.path.name)
            absent = sorted(set(weight_map) - set(where))
            if astray or absent:
                raise SafetensorsError(
                    "the index and the shards do not match: "
                    + "; ".join(part for part in (
                        f"not where the index says: {', '.join(astray[:8])}" if astray else "",
                        f"in the index but in no shard: {', '.join(absent[:8])}" if absent else "")
                        if part))
        bound = check_names(spec, stored)
        tensors = {}
        for name, (stored_name, axis) in bound.items():
            host = where[stored_name].tensor(stored_name)
            if axis is not None:
                host = host.squeeze(axis)
            kept = _kept_dtype(host.dtype, dtype)
            if host.is_floating_point() and not torch.isfinite(host.float()).all():
                raise ValueError(f"{stored_name} holds values that are not finite")
            tensors[name] = host.to(device=device, dtype=kept, copy=True)
        return tensors
    finally:
        for handle in files:
            handle.close()
