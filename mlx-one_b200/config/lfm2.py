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
        put = lambda name, value: object.__setattr__(self, name, value)
        if self.model_type != "lfm2":
            raise ConfigError(f"Lfm2Config cannot hold model_type={self.model_type!r}")
        for name in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "max_position_embeddings", "conv_L_cache",
                     "intermediate_size", "block_multiple_of"):
            positive_int(name, getattr(self, name))
        for name in ("norm_eps", "block_ffn_dim_multiplier", "rope_theta"):
            positive(name, getattr(self, name))
        for name in ("conv_bias", "block_auto_adjust_ff_dim", "block_use_swiglu",
                     "tie_embedding", "use_cache", "use_pos_enc"):
            boolean(name, getattr(self, name))
        divisible("hidden_size", self.hidden_size, "num_attention_heads",
                  self.num_attention_heads)
        divisible("num_attention_heads", self.num_attention_heads, "num_key_value_heads",
                  self.num_key_value_heads)
        if self.head_dim % 2:
            raise ConfigError("attention head dimension must be even for RoPE")
        if not self.block_use_swiglu:
            raise ConfigError("only SwiGLU LFM2 blocks are supported")
        if not self.use_pos_enc:
            raise ConfigError("LFM2 requires rotary positional encoding")
        block_dim = self.hidden_size if self.block_dim is None else self.block_dim
        if block_dim != self.hidden_size:
            raise ConfigError("block_dim must equal hidden_size")
        block_ff_dim = self.intermediate_size if self.block_ff_dim is None else self.block_ff_dim
        positive_int("block_ff_dim", block_ff_dim)
        if self.rope_parameters is not None:
            rope_type = self.rope_parameters.get("rope_type", "default")
            if rope_type != "default":
                raise ConfigError(f"unsupported LFM2 RoPE type: {rope_type}")
            theta = self.rope_parameters.get("rope_theta", self.rope_theta)
            positive("rope_theta", theta)
            put("rope_theta", float(theta))
        if self.layer_types is None:
            attention = set(self.full_attn_idxs if self.full_attn_idxs is not None
                            else range(3, self.num_hidden_layers, 4))
            layer_types = tuple("full_attention" if i in attention else "conv"
                                for i in range(self.num_hidden_layers))
        else:
            layer_types = tuple(self.layer_types)
        if len(layer_types) != self.num_hidden_layers:
            raise ConfigError("layer_types must contain one entry per hidden layer")
        for kind in layer_types:
            if kind not in LAYER_TYPES:
                raise ConfigError(f"unsupported LFM2 layer type: {kind}")
        attention_layers = tuple(i for i, kind in enumerate(layer_types)
                                 if kind in ATTENTION_TYPES)
        if not attention_layers:
            raise ConfigError("LFM2 requires at least one attention layer")
        if "sliding_attention" in layer_types:
            if self.sliding_window is None:
                raise ConfigError("sliding_attention requires sliding_window")
            positive_int("sliding_window", self.sliding_window)
        if self.full_attn_idxs is not None and tuple(self.full_attn_idxs) != attention_layers:
            raise ConfigError("full_attn_idxs must match layer_types")
        put("block_dim", block_dim)
        put("block_ff_dim", block_ff_dim)
        put("layer_types", layer_types)
        put("full_attn_idxs", attention_layers)
        put("rope_theta", float(self.rope_theta))
        put("norm_eps", float(self.norm_eps))

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

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Lfm2Config":
        data = dict(data)
        if "tie_embedding" not in data and "tie_word_embeddings" in data:
            data["tie_embedding"] = data["tie_word_embeddings"]
        if "num_attention_heads" not in data and "num_heads" in data:
            data["num_attention_heads"] = data["num_heads"]
        known = {item.name for item in fields(cls)} - {"extra"}
        payload = {key: value for key, value in data.items() if key in known}
        payload["extra"] = unknown_keys(data, known | {"tie_word_embeddings", "num_heads"})
        return cls(**payload)

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
