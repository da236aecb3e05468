"""Typed configuration of LFM2 (``Lfm2ForCausalLM``), read from its config.json keys.

Same fields, defaults, aliases, derivations and rejections as the reference's
``Lfm2Config`` (src/mlx_one/models/language/lfm2/config.py:12-155).
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Mapping, Sequence

from .base import ConfigError, boolean, divisible, positive, positive_int, unknown_keys

ATTENTION_TYPES = ("full_attention", "sliding_attention")
LAYER_TYPES = ("conv",) + ATTENTION_TYPES


@dataclass(frozen=True)
class Lfm2Config:
    model_type: str = "lfm2"
    vocab_size: int = 65536
    hidden_size: int = 1024
    num_hidden_layers: int = 16
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    max_position_embeddings: int = 128000
    norm_eps: float = 1e-5
    conv_bias: bool = False
    conv_L_cache: int = 3
    block_dim: int | None = None
    block_ff_dim: int | None = None
    intermediate_size: int = 6656
    block_multiple_of: int = 256
    block_ffn_dim_multiplier: float = 1.0
    block_auto_adjust_ff_dim: bool = True
    block_use_swiglu: bool = True
    layer_types: Sequence[str] | None = None
    full_attn_idxs: Sequence[int] | None = None
    rope_theta: float = 1_000_000.0
    rope_parameters: Mapping[str, Any] | None = None
    tie_embedding: bool = True
    use_cache: bool = True
    use_pos_enc: bool = True
    sliding_window: int | None = None
    eos_token_id: Any = None
    bos_token_id: Any = None
    extra: Mapping[str, Any] = field(default_factory=dict, repr=False)

    def __post_init__(self) -> None:
        if self.model_type != "lfm2":
            raise ConfigError(f"model_type {self.model_type!r} is not an LFM2 configuration")
        self._check_scalars()
        self._set(block_dim=self._block_dim(), block_ff_dim=self._block_ff_dim(),
                  rope_theta=self._theta(), norm_eps=float(self.norm_eps))
        kinds = self._layer_kinds()
        attention = tuple(i for i, kind in enumerate(kinds) if kind in ATTENTION_TYPES)
        if not attention:
            raise ConfigError("no layer of this LFM2 model attends; at least one has to")
        if "sliding_attention" in kinds:
            if self.sliding_window is None:
                raise ConfigError("a sliding_attention layer needs the key sliding_window")
            positive_int("sliding_window", self.sliding_window)
        if self.full_attn_idxs is not None and tuple(self.full_attn_idxs) != attention:
            raise ConfigError(f"full_attn_idxs {tuple(self.full_attn_idxs)} names other layers "
                              f"than layer_types does ({attention})")
        self._set(layer_types=kinds, full_attn_idxs=attention)

    def _set(self, **values: Any) -> None:
        for name, value in values.items():
            object.__setattr__(self, name, value)

    def _check_scalars(self) -> None:
        checks = {positive_int: ("vocab_size", "hidden_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads",
                                 "max_position_embeddings", "conv_L_cache", "intermediate_size",
                                 "block_multiple_of"),
                  positive: ("norm_eps", "block_ffn_dim_multiplier", "rope_theta"),
                  boolean: ("conv_bias", "block_auto_adjust_ff_dim", "block_use_swiglu",
                            "tie_embedding", "use_cache", "use_pos_enc")}
        for check, names in checks.items():
            for name in names:
                check(name, getattr(self, name))
        divisible("hidden_size", self.hidden_size, "num_attention_heads",
                  self.num_attention_heads)
        divisible("num_attention_heads", self.num_attention_heads, "num_key_value_heads",
                  self.num_key_value_heads)
        if self.head_dim % 2:
            raise ConfigError(f"head size {self.head_dim} is odd; the rotary encoding pairs "
                              f"dimensions")
        if not self.block_use_swiglu:
            raise ConfigError("block_use_swiglu=false: LFM2's feed-forward here is SwiGLU only")
        if not self.use_pos_enc:
            raise ConfigError("use_pos_enc=false: LFM2's attention here always rotates by "
                              "position")

    def _block_dim(self) -> int:
        if self.block_dim is not None and self.block_dim != self.hidden_size:
            raise ConfigError(f"block_dim ({self.block_dim}) differs from hidden_size "
                              f"({self.hidden_size})")
        return self.hidden_size

    def _block_ff_dim(self) -> int:
        width = self.intermediate_size if self.block_ff_dim is None else self.block_ff_dim
        positive_int("block_ff_dim", width)
        return width

    def _theta(self) -> float:
        theta = self.rope_theta
        if self.rope_parameters is not None:
            kind = self.rope_parameters.get("rope_type", "default")
            if kind != "default":
                raise ConfigError(f"rope_parameters.rope_type {kind!r}: only \"default\" is "
                                  f"implemented for LFM2")
            theta = self.rope_parameters.get("rope_theta", theta)
            positive("rope_parameters.rope_theta", theta)
        return float(theta)

    def _layer_kinds(self) -> tuple[str, ...]:
        """One kind per layer: given, or attention at ``full_attn_idxs`` (else at every fourth
        layer from the fourth) and convolution elsewhere."""
        if self.layer_types is not None:
            kinds = tuple(self.layer_types)
        else:
            where = (range(3, self.num_hidden_layers, 4) if self.full_attn_idxs is None
                     else self.full_attn_idxs)
            where = set(where)
            kinds = tuple("full_attention" if i in where else "conv"
                          for i in range(self.num_hidden_layers))
        if len(kinds) != self.num_hidden_layers:
            raise ConfigError(f"layer_types has {len(kinds)} entries for "
                              f"{self.num_hidden_layers} layers")
        strangers = sorted(set(kinds) - set(LAYER_TYPES))
        if strangers:
            raise ConfigError(f"layer_types names {strangers}; LFM2 layers are {LAYER_TYPES}")
        return kinds

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def adjusted_intermediate_size(self) -> int:
        """Width of the SwiGLU feed-forward (config.py:132-140 of the reference)."""
        if not self.block_auto_adjust_ff_dim:
            return int(self.block_ff_dim)
        width = int(2 * int(self.block_ff_dim) / 3)
        width = int(self.block_ffn_dim_multiplier * width)
        multiple = self.block_multiple_of
        return multiple * ((width + multiple - 1) // multiple)

    @property
    def eos_token_ids(self) -> tuple[int, ...]:
        eos = self.eos_token_id
        if eos is None:
            return ()
        return tuple(int(v) for v in eos) if isinstance(eos, (list, tuple)) else (int(eos),)

    # other spellings of a key that checkpoints use; the field's own name wins if both appear
    ALIASES = {"tie_word_embeddings": "tie_embedding", "num_heads": "num_attention_heads"}

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Lfm2Config":
        names = {item.name for item in fields(cls)} - {"extra"}
        values = {key: data[key] for key in names if key in data}
        for other, name in cls.ALIASES.items():
            if other in data:
                values.setdefault(name, data[other])
        return cls(**values, extra=unknown_keys(data, names | set(cls.ALIASES)))

    def to_dict(self) -> dict[str, Any]:
        """The config.json keys that describe this configuration."""
        out = {}
        for item in fields(self):
            if item.name == "extra":
                continue
            value = getattr(self, item.name)
            if value is None:
                continue
            out[item.name] = list(value) if isinstance(value, tuple) else value
        if isinstance(out.get("rope_parameters"), Mapping):
            out["rope_parameters"] = dict(out["rope_parameters"])
        out.update(self.extra)
        return out
