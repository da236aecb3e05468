"""Plain, slow LFM2 written from the reference's formulas.

The reference's model classes need ``mlx.nn`` and cannot be imported on this
machine, so this file rests on the formulas in its source, not on a run of it.
Every function cites the reference file and lines it restates (paths are
relative to the reference project's root).

Whole sequences only, no cache, one function per part. It shares no code with
the engine: it reads config.json keys and safetensors by itself.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# --------------------------------------------------------------------------- loading


def read_config(model_dir):
    """config.json as a plain dict, with the reference's defaults and aliases
    (src/mlx_one/models/language/lfm2/config.py:12-39, 142-155)."""
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    cfg = {
        "vocab_size": 65536, "hidden_size": 1024, "num_hidden_layers": 16,
        "num_attention_heads": 16, "num_key_value_heads": 8, "norm_eps": 1e-5,
        "conv_bias": False, "conv_L_cache": 3, "block_ff_dim": None,
        "intermediate_size": 6656, "block_multiple_of": 256,
        "block_ffn_dim_multiplier": 1.0, "block_auto_adjust_ff_dim": True,
        "layer_types": None, "full_attn_idxs": None, "rope_theta": 1_000_000.0,
        "rope_parameters": None, "tie_embedding": True, "sliding_window": None,
    }
    if "tie_embedding" not in raw and "tie_word_embeddings" in raw:
        raw["tie_embedding"] = raw["tie_word_embeddings"]
    if "num_attention_heads" not in raw and "num_heads" in raw:
        raw["num_attention_heads"] = raw["num_heads"]
    for key in cfg:
        if key in raw:
            cfg[key] = raw[key]
    if cfg["rope_parameters"]:
        cfg["rope_theta"] = float(cfg["rope_parameters"].get("rope_theta", cfg["rope_theta"]))
    if cfg["block_ff_dim"] is None:
        cfg["block_ff_dim"] = cfg["intermediate_size"]
    if cfg["layer_types"] is None:
        # config.py:85-95: attention at full_attn_idxs, else at range(3, L, 4)
        layers = cfg["num_hidden_layers"]
        attention = set(cfg["full_attn_idxs"] if cfg["full_attn_idxs"] is not None
                        else range(3, layers, 4))
        cfg["layer_types"] = ["full_attention" if i in attention else "conv"
                              for i in range(layers)]
    return cfg


def feed_forward_width(cfg):
    """src/mlx_one/models/language/lfm2/config.py:132-140."""
    if not cfg["block_auto_adjust_ff_dim"]:
        return int(cfg["block_ff_dim"])
    width = int(2 * int(cfg["block_ff_dim"]) / 3)
    width = int(cfg["block_ffn_dim_multiplier"] * width)
    multiple = cfg["block_multiple_of"]
    return multiple * ((width + multiple - 1) // multiple)


def read_weights(model_dir, dtype=torch.float32):
    """All tensors of model.safetensors, renamed as the reference's sanitizer does
    (src/mlx_one/models/language/lfm2/weights.py:11-26), promoted to ``dtype``."""
    from safetensors.torch import load_file

    tensors = {}
    for name, value in load_file(str(Path(model_dir) / "model.safetensors")).items():
        if name.endswith(("rotary_emb.inv_freq", "position_ids")):
            continue
        if name.endswith("conv.conv.weight"):
            name = name[: -len(".weight")]
        if name.endswith("conv.conv.bias"):
            name = name[: -len("conv.bias")] + "conv_bias"
        if name.endswith("conv.conv") and value.dim() == 3:
            value = value[:, :, 0] if value.shape[-1] == 1 else value[:, 0, :]
        tensors[name] = value.to(dtype)
    return tensors


# --------------------------------------------------------------------------- parts


def rms_norm(x, weight, eps):
    """v * rsqrt(mean(v^2) + eps) * w over the last axis, plain weight.
    nn.RMSNorm as used at src/mlx_one/models/language/lfm2/reference_math.py:64-65,156-157;
    the formula is spelled out at src/mlx_one/models/vision_language/qwen3_5/model.py:53-54."""
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(variance + eps) * weight


def rope_angles(positions, head_dim, theta):
    """inv_freq_j = theta^(-j/(hd/2)); angle = position * inv_freq, in 32-bit
    (src/mlx_one/models/shared/transformer.py:50-51, 67-72)."""
    half = head_dim // 2
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=torch.float32),
                         -torch.arange(half, dtype=torch.float32) / half)
    return positions.to(torch.float32)[:, None] * inv_freq[None, :]


def apply_rope(x, angles):
    """Non-interleaved rotation of all head dims: value*cos + rotate_half(value)*sin with
    rotate_half = concat(-second half, first half)
    (src/mlx_one/models/shared/transformer.py:27-29, 88-90). x: [T, heads, hd]."""
    cos = torch.cos(angles).to(x.dtype)[:, None, :]
    sin = torch.sin(angles).to(x.dtype)[:, None, :]
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)


def short_conv_mixer(n, w, prefix, cfg):
    """Gated short convolution over a whole sequence from position 0
    (src/mlx_one/models/language/lfm2/reference_math.py:36-49): in_proj, split into
    B, C, x, B*x, zero left padding of L-1 rows, depthwise causal conv where the last
    tap multiplies the current token, bias, C*y, out_proj."""
    taps = cfg["conv_L_cache"]
    bcx = n @ w[prefix + "conv.in_proj.weight"].T
    if cfg["conv_bias"]:
        bcx = bcx + w[prefix + "conv.in_proj.bias"]
    gate_b, gate_c, x = bcx.chunk(3, dim=-1)
    g = gate_b * x
    padded = torch.cat((g.new_zeros(taps - 1, g.shape[1]), g), dim=0)
    kernel = w[prefix + "conv.conv"]  # [H, taps]
    y = torch.zeros_like(g)
    for k in range(taps):
        y = y + padded[k:k + g.shape[0]] * kernel[:, k]
    if cfg["conv_bias"]:
        y = y + w[prefix + "conv.conv_bias"]
    out = (gate_c * y) @ w[prefix + "conv.out_proj.weight"].T
    if cfg["conv_bias"]:
        out = out + w[prefix + "conv.out_proj.bias"]
    return out


def attention_mixer(n, w, prefix, cfg, window=None):
    """Grouped-query attention over a whole sequence from position 0
    (src/mlx_one/models/language/lfm2/reference_math.py:85-111): q/k/v projections,
    per-head RMSNorm of q and k before RoPE, RoPE, causal softmax(q k^T hd^-0.5) v with
    query head h reading key head h // (heads / kv_heads), out_proj. A window keeps
    keys with key > query - window (src/mlx_one/models/shared/hybrid.py:14-20)."""
    tokens = n.shape[0]
    heads, kv_heads = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    head_dim = cfg["hidden_size"] // heads
    q = (n @ w[prefix + "self_attn.q_proj.weight"].T).view(tokens, heads, head_dim)
    k = (n @ w[prefix + "self_attn.k_proj.weight"].T).view(tokens, kv_heads, head_dim)
    v = (n @ w[prefix + "self_attn.v_proj.weight"].T).view(tokens, kv_heads, head_dim)
    q = rms_norm(q, w[prefix + "self_attn.q_layernorm.weight"], cfg["norm_eps"])
    k = rms_norm(k, w[prefix + "self_attn.k_layernorm.weight"], cfg["norm_eps"])
    angles = rope_angles(torch.arange(tokens), head_dim, cfg["rope_theta"])
    q, k = apply_rope(q, angles), apply_rope(k, angles)
    out = causal_attention(q, k, v, window)
    return out.reshape(tokens, heads * head_dim) @ w[prefix + "self_attn.out_proj.weight"].T


def causal_attention(q, k, v, window=None):
    """softmax(q k^T hd^-0.5) v over a whole sequence from position 0, the query at position t
    seeing keys at positions <= t (and > t - window); query head h reads key head
    h // (heads / kv_heads) (src/mlx_one/engine/paged_attention.py:104-105, 222-226 for the
    mapping and the bound). q: [T, heads, hd]; k, v: [T, kv_heads, hd]; returns [T, heads, hd]."""
    tokens, heads, head_dim = q.shape
    group = heads // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, k) * head_dim ** -0.5
    query = torch.arange(tokens)[:, None]
    key = torch.arange(tokens)[None, :]
    allowed = key <= query
    if window is not None:
        allowed = allowed & (key > query - window)
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), v)


def swiglu_feed_forward(n, w, prefix):
    """w2(silu(w1 n) * w3 n) (src/mlx_one/models/language/lfm2/reference_math.py:134-135;
    src/mlx_one/models/shared/reference_activations.py:11-13)."""
    gate = n @ w[prefix + "feed_forward.w1.weight"].T
    up = n @ w[prefix + "feed_forward.w3.weight"].T
    return (torch.nn.functional.silu(gate) * up) @ w[prefix + "feed_forward.w2.weight"].T


def decoder_layer(x, w, index, cfg):
    """h = x + mixer(operator_norm(x)); out = h + ffn(ffn_norm(h))
    (src/mlx_one/models/language/lfm2/reference_math.py:160-179)."""
    prefix = f"model.layers.{index}."
    kind = cfg["layer_types"][index]
    n = rms_norm(x, w[prefix + "operator_norm.weight"], cfg["norm_eps"])
    if kind == "conv":
        r = short_conv_mixer(n, w, prefix, cfg)
    else:
        window = cfg["sliding_window"] if kind == "sliding_attention" else None
        r = attention_mixer(n, w, prefix, cfg, window)
    h = x + r
    return h + swiglu_feed_forward(rms_norm(h, w[prefix + "ffn_norm.weight"], cfg["norm_eps"]),
                                   w, prefix)


def forward(cfg, w, token_ids):
    """Logits [T, V] of one whole sequence (src/mlx_one/models/language/lfm2/model.py:48-82,
    120-124): embedding, layers, embedding_norm, tied or separate head."""
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    x = w["model.embed_tokens.weight"][ids]
    for index in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, index, cfg)
    x = rms_norm(x, w["model.embedding_norm.weight"], cfg["norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_embedding"] else w["lm_head.weight"]
    return x @ head.T


class PlainModel:
    """A model folder read by the plain implementation."""

    def __init__(self, model_dir, dtype=torch.float32):
        self.cfg = read_config(model_dir)
        self.w = read_weights(model_dir, dtype)

    @torch.no_grad()
    def logits(self, token_ids):
        return forward(self.cfg, self.w, token_ids)

    @torch.no_grad()
    def greedy(self, prompt, count):
        """Greedy continuation by recomputing the whole sequence for each token."""
        ids = list(prompt)
        for _ in range(count):
            ids.append(int(torch.argmax(self.logits(ids)[-1])))
        return ids[len(prompt):]


# --------------------------------------------------------------------------- sampling


def sample_token(logits, temperature, top_k, top_p, uniform):
    """The reference's selection rule with the random number given
    (src/mlx_one/text/sampling.py:37-88): greedy at temperature 0; else softmax(logits/T),
    stable descending order (ties by token id), keep top_k, keep the shortest prefix whose
    mass reaches top_p * kept mass, draw uniform * kept mass and take the first rank whose
    cumulative mass reaches it."""
    logits = torch.as_tensor(logits, dtype=torch.float64)
    if temperature == 0:
        return int(torch.argmax(logits))
    p = torch.softmax(logits / temperature, dim=-1)
    order = torch.sort(p, descending=True, stable=True).indices
    if top_k is not None:
        order = order[:top_k]
    ranked = p[order]
    cumulative = torch.cumsum(ranked, dim=0)
    if top_p < 1.0:
        cutoff = top_p * float(ranked.sum())
        count = min(int(torch.searchsorted(cumulative, torch.tensor(cutoff, dtype=torch.float64),
                                           right=False)) + 1, len(order))
        order, ranked, cumulative = order[:count], ranked[:count], cumulative[:count]
    threshold = uniform * float(ranked.sum())
    index = min(int(torch.searchsorted(cumulative, torch.tensor(threshold, dtype=torch.float64),
                                       right=False)), len(order) - 1)
    return int(order[index])


def counter_uniform(seed, step):
    """The engine's documented per-request random number: a splitmix64 hash of
    (seed, step) mapped to [0, 1) with 24 bits. Not from the reference (it uses
    Python's Mersenne Twister on the host); restated here from the engine's
    documentation so that the test does not import the engine's sampler."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + (step + 1) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)
