"""Sequence mixers: grouped-query attention over paged keys and values, and the gated
short convolution with a fixed-size state."""

from __future__ import annotations

import torch

from .base import FixedState, Mixer, PagedKeyValues
from .registry import MIXERS, POSITIONS
from .spec import PartSpec, TensorSpec


@MIXERS.register("attention")
class Attention(Mixer):
    """Grouped-query attention. Parameters: ``hidden``, ``heads``, ``kv_heads``,
    ``head_dim``, ``qk_norm_eps`` (None = no per-head RMSNorm of queries and keys),
    ``position`` (a position-encoding PartSpec), ``window`` (None = all keys),
    ``scale`` (None = head_dim^-0.5).

    q, k, v projections (one fused matrix product), per-head RMSNorm of q and k, rotation,
    keys and values appended to the request's pages, causal softmax(q k^T scale) v where
    query head h reads key head h // (heads / kv_heads), output projection.
    Reference: src/mlx_one/models/language/lfm2/reference_math.py:52-111; window mask
    src/mlx_one/models/shared/hybrid.py:14-20."""

    @classmethod
    def tensors(cls, spec):
        hidden, hd = spec["hidden"], spec["head_dim"]
        q_dim, kv_dim = spec["heads"] * hd, spec["kv_heads"] * hd
        out = {
            "q_proj.weight": TensorSpec((q_dim, hidden)),
            "k_proj.weight": TensorSpec((kv_dim, hidden)),
            "v_proj.weight": TensorSpec((kv_dim, hidden)),
            "out_proj.weight": TensorSpec((hidden, q_dim)),
        }
        if spec.get("qk_norm_eps") is not None:
            out["q_layernorm.weight"] = TensorSpec((hd,), "norm")
            out["k_layernorm.weight"] = TensorSpec((hd,), "norm")
        return out

    @classmethod
    def cache_need(cls, spec):
        return PagedKeyValues(spec["kv_heads"], spec["head_dim"], spec.get("window"))

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.heads, self.kv_heads, self.head_dim = spec["heads"], spec["kv_heads"], spec["head_dim"]
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.window = spec.get("window")
        scale = spec.get("scale")
        self.scale = float(self.head_dim ** -0.5 if scale is None else scale)
        self.qkv = self.matrix(torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                          tensors["v_proj.weight"]], dim=0))
        self.out = self.matrix(tensors["out_proj.weight"])
        self.eps = spec.get("qk_norm_eps")
        self.q_norm = self.k_norm = None
        if self.eps is not None:
            self.q_norm = self.vector(tensors["q_layernorm.weight"])
            self.k_norm = self.vector(tensors["k_layernorm.weight"])
        position: PartSpec = spec.get("position") or PartSpec("none")
        self.position = POSITIONS.get(position.kind)(position, {}, runtime)
        self.ops.check_attention_sizes(self.heads, self.kv_heads, self.head_dim)

    fuses_residual = True
    accepts_normed_input = True

    def forward(self, x, ctx, cache, write, residual=None):
        qkv = self.ops.linear(x, self.qkv)
        mixed = self.ops.qkv_attention(
            qkv, heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim,
            q_weight=self.q_norm, k_weight=self.k_norm, eps=self.eps,
            rotary=self.position.rotary_table(), scale=self.scale, window=self.window, ctx=ctx,
            view=cache, write=write)
        if residual is None:
            return self.ops.linear(mixed, self.out)
        return self.ops.linear_add(mixed, self.out, None, residual)


@MIXERS.register("short_conv")
class ShortConv(Mixer):
    """Gated short convolution. Parameters: ``hidden``, ``taps`` (kernel width), ``bias``.

    BCx = in_proj(x) split in the order B, C, x; g = B * x; y[t] = sum_k conv[:, k] *
    g[t - (taps-1) + k] over this request's tokens (zero before its first token), + bias;
    output = out_proj(C * y). The state is the last taps-1 rows of g.
    Reference: src/mlx_one/models/language/lfm2/reference_math.py:19-49; state
    src/mlx_one/core/cache.py:476-491; batched carry src/mlx_one/engine/hybrid.py:67-82."""

    @classmethod
    def tensors(cls, spec):
        hidden, taps = spec["hidden"], spec["taps"]
        out = {
            "in_proj.weight": TensorSpec((3 * hidden, hidden)),
            "conv": TensorSpec((hidden, taps)),
            "out_proj.weight": TensorSpec((hidden, hidden)),
        }
        if spec.get("bias"):
            out["in_proj.bias"] = TensorSpec((3 * hidden,), "bias")
            out["conv_bias"] = TensorSpec((hidden,), "bias")
            out["out_proj.bias"] = TensorSpec((hidden,), "bias")
        return out

    @classmethod
    def cache_need(cls, spec):
        return FixedState((max(spec["taps"] - 1, 1), spec["hidden"]))

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.hidden, self.taps = spec["hidden"], spec["taps"]
        self.in_proj = self.matrix(tensors["in_proj.weight"])
        self.out_proj = self.matrix(tensors["out_proj.weight"])
        self.kernel = self.vector(tensors["conv"])
        bias = bool(spec.get("bias"))
        self.in_bias = self.vector(tensors["in_proj.bias"]) if bias else None
        self.conv_bias = self.vector(tensors["conv_bias"]) if bias else None
        self.out_bias = self.vector(tensors["out_proj.bias"]) if bias else None

    fuses_residual = True
    accepts_normed_input = True

    def forward(self, x, ctx, cache, write, residual=None):
        gated = self.ops.linear_short_conv(x, self.in_proj, self.in_bias, kernel=self.kernel,
                                           bias=self.conv_bias, taps=self.taps, ctx=ctx,
                                           view=cache, write=write)
        if residual is None:
            return self.ops.linear(gated, self.out_proj, self.out_bias)
        return self.ops.linear_add(gated, self.out_proj, self.out_bias, residual)
