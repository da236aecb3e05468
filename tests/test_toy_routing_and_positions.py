"""Two more toy parts defined here, in the test, and registered without a change to the
framework's files: a feed-forward that routes every token to one of several small experts
(router logits in 32-bit), and a position encoding of its own (rotation of a part of the head
only, with positions stretched by a factor). They are built into a toy architecture next to the
framework's attention and norms, loaded from a folder with random weights and stepped through the
engine's loader, cache manager and step function in portions and single tokens."""

import dataclasses

import pytest
import torch

from mlx_one_b200.cache import CacheManager
from mlx_one_b200.config import Architecture, register_architecture, unregister_architecture
from mlx_one_b200.engine.loading import load_model
from mlx_one_b200.engine.runner import Runner
from mlx_one_b200.parts import (FEED_FORWARDS, POSITIONS, FeedForward, LayerCall, LayerSpec,
                                ModelSpec, PartSpec, PositionEncoding, TensorSpec)
from mlx_one_b200.weights import write_random_model
from plain_lfm2 import rms_norm
from tiny_models import assert_close, cut, prompts, replay


@dataclasses.dataclass(frozen=True)
class RoutedConfig:
    model_type: str = "toy-routed"
    vocab_size: int = 131
    hidden_size: int = 64
    heads: int = 4
    kv_heads: int = 2
    experts: int = 3
    expert_width: int = 40
    rotary_dim: int = 8            # of a head size of 16
    stretch: float = 4.0
    theta: float = 500.0
    layers: int = 2
    eps: float = 1e-5

    @classmethod
    def from_dict(cls, data):
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in data.items() if k in names})

    def to_dict(self):
        return dataclasses.asdict(self)


class RoutedFeedForward(FeedForward):
    """Every token goes to the expert with the largest router logit (logits in 32-bit); the
    expert is w_out(gelu(w_in x)), scaled by the sigmoid of its logit. The router is made
    decisive (its weights are scaled up) so that rounding does not change a token's expert."""

    # the rows of an expert are found with nonzero(), which waits for the device and gives
    # tensors whose sizes depend on the data: such a step cannot be replayed from a graph
    capturable = False

    @classmethod
    def tensors(cls, spec):
        hidden, width = spec["hidden"], spec["width"]
        out = {"router.weight": TensorSpec((spec["experts"], hidden))}
        for e in range(spec["experts"]):
            out[f"experts.{e}.w_in.weight"] = TensorSpec((width, hidden))
            out[f"experts.{e}.w_out.weight"] = TensorSpec((hidden, width))
        return out

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.router = tensors["router.weight"].float() * 200
        self.experts = [(self.matrix(tensors[f"experts.{e}.w_in.weight"]),
                         self.matrix(tensors[f"experts.{e}.w_out.weight"]))
                        for e in range(spec["experts"])]

    def forward(self, x, ctx):
        logits = x.float() @ self.router.T                    # [tokens, experts], 32-bit
        choice = logits.argmax(dim=-1)
        out = torch.zeros_like(x)
        for e, (w_in, w_out) in enumerate(self.experts):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel() == 0:
                continue
            hidden = torch.nn.functional.gelu(self.ops.linear(x[rows].contiguous(), w_in).float())
            gate = torch.sigmoid(logits[rows, e])[:, None]
            expert = self.ops.linear(hidden.to(x.dtype), w_out).float() * gate
            out[rows] = expert.to(x.dtype)
        return out


class StretchedPartialRotation(PositionEncoding):
    """Rotates the first ``rotary_dim`` dimensions of a head only, by position / stretch."""

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        half = spec["rotary_dim"] // 2
        inv_freq = torch.pow(torch.tensor(float(spec["theta"])),
                             -torch.arange(half, dtype=torch.float32) / half) / spec["stretch"]
        self.inv_freq, self.rotary_dim = inv_freq.to(runtime.device), spec["rotary_dim"]

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim


def describe(config: RoutedConfig) -> ModelSpec:
    hidden, head_dim = config.hidden_size, config.hidden_size // config.heads
    norm = lambda prefix: PartSpec("rmsnorm", {"size": hidden, "eps": config.eps}, prefix)
    position = PartSpec("toy_stretched_rotation", {"theta": config.theta, "stretch": config.stretch,
                                                   "rotary_dim": config.rotary_dim})
    attention = PartSpec("attention", {"hidden": hidden, "heads": config.heads,
                                       "kv_heads": config.kv_heads, "head_dim": head_dim,
                                       "qk_norm_eps": None, "position": position, "window": None,
                                       "scale": None}, "attn.")
    routed = PartSpec("toy_routed", {"hidden": hidden, "width": config.expert_width,
                                     "experts": config.experts}, "moe.")
    layers = tuple(LayerSpec(f"layers.{i}.", PartSpec("prenorm"), attention, norm("norm1."), routed,
                             norm("norm2.")) for i in range(config.layers))
    return ModelSpec(architecture="toy-routed", vocab_size=config.vocab_size, hidden_size=hidden,
                     embedding="embed.weight", layers=layers,
                     order=tuple(LayerCall(i) for i in range(config.layers)),
                     final_norm=norm("final_norm."), head="head.weight", max_positions=4096)


def plain_routed(w, cfg: RoutedConfig, ids):
    """The same model over a whole sequence, written out plainly."""
    tokens, hd = len(ids), cfg.hidden_size // cfg.heads
    x = w["embed.weight"][torch.tensor(ids)]
    half = cfg.rotary_dim // 2
    inv_freq = torch.pow(torch.tensor(cfg.theta), -torch.arange(half, dtype=torch.float32) / half)
    angles = torch.arange(tokens, dtype=torch.float32)[:, None] * (inv_freq / cfg.stretch)[None, :]

    def rotate(t):                                   # [tokens, heads, hd]: the first dims only
        a, b, rest = t[..., :half], t[..., half:cfg.rotary_dim], t[..., cfg.rotary_dim:]
        cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
        return torch.cat((a * cos - b * sin, b * cos + a * sin, rest), dim=-1)

    for layer in range(cfg.layers):
        p = f"layers.{layer}."
        n = rms_norm(x, w[p + "norm1.weight"], cfg.eps)
        q = rotate((n @ w[p + "attn.q_proj.weight"].T).view(tokens, cfg.heads, hd))
        k = rotate((n @ w[p + "attn.k_proj.weight"].T).view(tokens, cfg.kv_heads, hd))
        v = (n @ w[p + "attn.v_proj.weight"].T).view(tokens, cfg.kv_heads, hd)
        group = cfg.heads // cfg.kv_heads
        scores = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(group, 1)) * hd ** -0.5
        mask = torch.arange(tokens)[None, :] <= torch.arange(tokens)[:, None]
        scores = scores.masked_fill(~mask[None], float("-inf"))
        mixed = torch.einsum("hqk,khd->qhd", torch.softmax(scores, -1), v.repeat_interleave(group, 1))
        h = x + mixed.reshape(tokens, -1) @ w[p + "attn.out_proj.weight"].T
        n = rms_norm(h, w[p + "norm2.weight"], cfg.eps)
        logits = n @ (w[p + "moe.router.weight"] * 200).T
        choice = logits.argmax(-1)
        out = torch.zeros_like(n)
        for t in range(tokens):
            e = int(choice[t])
            inner = torch.nn.functional.gelu(n[t] @ w[p + f"moe.experts.{e}.w_in.weight"].T)
            out[t] = (inner @ w[p + f"moe.experts.{e}.w_out.weight"].T) * torch.sigmoid(logits[t, e])
        x = h + out
    return rms_norm(x, w["final_norm.weight"], cfg.eps) @ w["head.weight"].T


@pytest.fixture()
def routed_registered():
    FEED_FORWARDS.register("toy_routed", RoutedFeedForward)
    POSITIONS.register("toy_stretched_rotation", StretchedPartialRotation)
    register_architecture(Architecture("toy-routed", RoutedConfig, describe))
    yield
    unregister_architecture("toy-routed")
    POSITIONS.unregister("toy_stretched_rotation")
    FEED_FORWARDS.unregister("toy_routed")


def run_routed(tmp_path, device, ops):
    cfg = RoutedConfig()
    folder = write_random_model(tmp_path / "routed", cfg.to_dict(), seed=11, dtype=torch.float32)
    loaded = load_model(folder, torch.float32, device, ops=ops)
    model = loaded.model
    cache = CacheManager(model.cache_needs, page_size=8, capacity_tokens=128, max_requests=3,
                         dtype=model.runtime.dtype, device=device)
    runner = Runner(model, cache)
    from safetensors.torch import load_file
    weights = {k: v.float() for k, v in load_file(str(folder / "model.safetensors")).items()}
    requests = prompts(cfg.vocab_size, (29, 41), seed=2)
    steps = [([(0, part)], []) for part in cut(requests[0], (7, 2, 11))]
    steps += [([(1, requests[1][:25])], [])]
    steps += [([(1, [t])], []) for t in requests[1][25:]]
    got = replay(runner, cache, steps)
    for i, tokens in enumerate(requests):
        assert_close(got[i], plain_routed(weights, cfg, tokens), torch.float32, f"routed {i}")
    used = set()
    hidden = weights["embed.weight"][torch.tensor(requests[1])]
    for layer in range(cfg.layers):
        # (a rough look at the router over the embeddings: more than one expert is in play)
        logits = rms_norm(hidden, weights[f"layers.{layer}.norm2.weight"], cfg.eps) @ \
            weights[f"layers.{layer}.moe.router.weight"].T
        used |= set(logits.argmax(-1).tolist())
    assert len(used) > 1


def test_routed_architecture_on_the_cpu(tmp_path, routed_registered):
    from plain_ops import PlainOps
    run_routed(tmp_path, "cpu", PlainOps())


@pytest.mark.gpu
def test_routed_architecture_on_the_gpu(tmp_path, routed_registered):
    run_routed(tmp_path, "cuda:0", None)
