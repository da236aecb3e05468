"""LFM2 (``Lfm2ForCausalLM``) described in parts.

Every layer is a pre-norm block with a SwiGLU feed-forward; the mixer is the gated short
convolution for ``conv`` layers and grouped-query attention with per-head q/k RMSNorm and
rotary encoding for ``full_attention`` and ``sliding_attention`` layers.
Reference: src/mlx_one/models/language/lfm2/model.py:26-125,
src/mlx_one/models/language/lfm2/reference_math.py:138-179; tensor names and shapes
src/mlx_one/models/language/lfm2/weights.py:29-78.
"""

from __future__ import annotations

from ..config.lfm2 import Lfm2Config
from ..config.registry import Architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def rename_tensor(name: str, shape: tuple[int, ...]):
    """Stored name -> (engine name, axis to squeeze) or None to drop it
    (src/mlx_one/models/language/lfm2/weights.py:11-26). The depthwise kernel may be stored
    as ``conv.conv.weight`` of shape [H, 1, L] or [H, L, 1]; its bias as ``conv.conv.bias``."""
    if name.endswith(("rotary_emb.inv_freq", "position_ids")):
        return None
    axis = None
    if name.endswith("conv.conv.weight"):
        name = name[: -len(".weight")]
    elif name.endswith("conv.conv.bias"):
        name = name[: -len("conv.bias")] + "conv_bias"
    if name.endswith("conv.conv") and len(shape) == 3:
        if shape[-1] == 1:
            axis = 2
        elif shape[1] == 1:
            axis = 1
    return name, axis


def describe(config: Lfm2Config) -> ModelSpec:
    hidden = config.hidden_size
    norm = lambda prefix: PartSpec("rmsnorm", {"size": hidden, "eps": config.norm_eps}, prefix)
    feed_forward = PartSpec("swiglu", {"hidden": hidden,
                                       "width": config.adjusted_intermediate_size},
                            "feed_forward.")
    rope = PartSpec("rope", {"theta": config.rope_theta, "rotary_dim": config.head_dim})
    layers = []
    for index, kind in enumerate(config.layer_types):
        if kind == "conv":
            mixer = PartSpec("short_conv", {"hidden": hidden, "taps": config.conv_L_cache,
                                            "bias": config.conv_bias}, "conv.")
        else:
            mixer = PartSpec("attention", {
                "hidden": hidden, "heads": config.num_attention_heads,
                "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                "qk_norm_eps": config.norm_eps, "position": rope, "scale": None,
                "window": config.sliding_window if kind == "sliding_attention" else None,
            }, "self_attn.")
        layers.append(LayerSpec(
            prefix=f"model.layers.{index}.", block=PartSpec("prenorm"), mixer=mixer,
            mixer_norm=norm("operator_norm."), feed_forward=feed_forward,
            feed_forward_norm=norm("ffn_norm.")))
    bos = config.bos_token_id
    return ModelSpec(
        architecture="lfm2", vocab_size=config.vocab_size, hidden_size=hidden,
        embedding="model.embed_tokens.weight", layers=tuple(layers),
        order=tuple(LayerCall(index) for index in range(len(layers))),
        final_norm=norm("model.embedding_norm."),
        head=None if config.tie_embedding else "lm_head.weight",
        max_positions=config.max_position_embeddings,
        eos_token_ids=config.eos_token_ids,
        bos_token_id=None if bos is None else int(bos),
        rename=(lambda name, shape: None if config.tie_embedding and name == "lm_head.weight"
                else rename_tensor(name, shape)))


ARCHITECTURE = Architecture("lfm2", Lfm2Config, describe)
