"""What a caller may ask of a generation, and what comes back.

The field names, their defaults and their meanings are the reference's
(src/mlx_one/text/schemas.py:10-70), so that code written for its ``TextGenerationOptions``,
``GenerationChunk`` and ``GenerationResult`` reads the same here. The checks are a table of
(field, rule) pairs, one line per field, evaluated when the options are made.
"""

from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import Any, Callable


def _is_int(value: Any) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def _is_real(value: Any) -> bool:
    return isinstance(value, (int, float)) and not isinstance(value, bool)


# field -> (what a good value looks like, in words; the test that says so)
_RULES: dict[str, tuple[str, Callable[[Any], bool]]] = {
    "max_tokens": ("an integer of at least 1", lambda v: _is_int(v) and v >= 1),
    "temperature": ("a number of at least 0 (0 means greedy)", lambda v: _is_real(v) and v >= 0),
    "top_k": ("None or an integer of at least 1", lambda v: v is None or (_is_int(v) and v >= 1)),
    "top_p": ("a number above 0 and at most 1", lambda v: _is_real(v) and 0 < v <= 1),
    "seed": ("an integer", _is_int),
    "stop": ("a sequence of strings, none of them empty",
             lambda v: not isinstance(v, str) and all(isinstance(s, str) and s for s in v)),
    "ignore_eos": ("a boolean", lambda v: isinstance(v, bool)),
}


@dataclass(frozen=True)
class TextGenerationOptions:
    max_tokens: int = 128
    temperature: float = 0.0        # 0 = greedy
    top_k: int | None = None
    top_p: float = 1.0
    seed: int = 0
    stop: tuple[str, ...] = ()
    ignore_eos: bool = False        # keep decoding past end-of-sequence tokens (benchmarks)

    def __post_init__(self) -> None:
        for name, (wanted, good) in _RULES.items():
            value = getattr(self, name)
            try:
                accepted = good(value)
            except TypeError:
                accepted = False
            if not accepted:
                raise ValueError(f"option {name}={value!r}: expected {wanted}")
        # normalised forms: floats as floats, stop strings as a tuple
        for name, as_type in (("temperature", float), ("top_p", float), ("stop", tuple)):
            object.__setattr__(self, name, as_type(getattr(self, name)))

    def replace(self, **changes: Any) -> "TextGenerationOptions":
        return dataclasses.replace(self, **changes)


@dataclass(frozen=True)
class GenerationChunk:
    token_id: int | None
    text: str
    generated_tokens: int
    finish_reason: str | None = None         # "stop" | "length" | None while running
    terminal_token_id: int | None = None


@dataclass(frozen=True)
class GenerationResult:
    prompt: str
    text: str
    prompt_tokens: int
    generation_tokens: int
    finish_reason: str
    model: str
    revision: str | None = None
    timings: dict[str, float] = field(default_factory=dict)
    token_ids: tuple[int, ...] = ()

    def to_dict(self) -> dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), sort_keys=True, indent=2)
