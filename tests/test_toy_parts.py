"""A toy architecture defined here, in the test: a mixer with fixed-size state of its own, a
layer that runs twice, and a call that reads another call's cache. It is registered, built,
loaded from a folder with random weights and stepped through the engine's own loader, cache
manager and step function, with no change to the framework's files, on the CPU (plain kernel
restatements) and on the GPU (CUDA kernels for every part that is the framework's)."""

import dataclasses
import json

import pytest
import torch

from mlx_one_b200.cache import CacheManager
from mlx_one_b200.config import Architecture, register_architecture, unregister_architecture
from mlx_one_b200.engine.loading import load_model
from mlx_one_b200.engine.runner import Runner
from mlx_one_b200.parts import (MIXERS, FixedState, LayerCall, LayerSpec, Mixer, ModelSpec,
                                PartSpec, TensorSpec)
from mlx_one_b200.weights import write_random_model
from plain_lfm2 import apply_rope, rms_norm, rope_angles
from tiny_models import assert_close, cut, prompts, replay


@dataclasses.dataclass(frozen=True)
class ToyConfig:
    model_type: str = "toy-decay"
    vocab_size: int = 97
    hidden_size: int = 48
    heads: int = 3
    kv_heads: int = 1
    width: int = 80
    eps: float = 1e-5

    @classmethod
    def from_dict(cls, data):
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in data.items() if k in names})

    def to_dict(self):
        return dataclasses.asdict(self)


class DecayMixer(Mixer):
    """s_t = a * s_{t-1} + (1 - a) * x_t per channel, a = sigmoid(decay); out = W s_t.
    The state s is kept per request in a slot, in 32-bit."""

    # forward loops over the requests on the host (ctx.host, .tolist()): not for CUDA graphs
    capturable = False

    @classmethod
    def tensors(cls, spec):
        hidden = spec["hidden"]
        return {"decay": TensorSpec((hidden,), "bias"), "mix.weight": TensorSpec((hidden, hidden))}

    @classmethod
    def cache_need(cls, spec):
        return FixedState((spec["hidden"],), dtype="float32")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.rate = torch.sigmoid(tensors["decay"].float() * 50)
        self.mix = self.matrix(tensors["mix.weight"])

    def forward(self, x, ctx, cache, write):
        out = torch.empty_like(x, dtype=torch.float32)
        starts = ctx.host["request_start"]
        slots = cache.slots.tolist()
        for r in range(ctx.requests):
            state = cache.state[slots[r]].clone()
            for t in range(starts[r], starts[r + 1]):
                state = self.rate * state + (1 - self.rate) * x[t].float()
                out[t] = state
            if write:
                cache.state[slots[r]] = state
        return self.ops.linear(out.to(x.dtype), self.mix)


class ShiftMixer(Mixer):
    """out_t = W (x_t + x_{t-1}), where x_{t-1} is the request's previous token (zero before
    its first). The state is the request's last input row. Written with torch operations on
    the step's device tensors only (no host value, no wait), so its steps can be captured as
    CUDA graphs and replayed with another split of the tokens."""

    @classmethod
    def tensors(cls, spec):
        return {"mix.weight": TensorSpec((spec["hidden"], spec["hidden"]))}

    @classmethod
    def cache_need(cls, spec):
        return FixedState((spec["hidden"],), dtype="float32")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.mix = self.matrix(tensors["mix.weight"])

    def forward(self, x, ctx, cache, write):
        owner = ctx.token_request.long()
        first = ctx.positions == ctx.history[owner]             # a request's first token here
        before = torch.roll(x.float(), 1, dims=0)
        carried = cache.state[cache.slots.long()][owner]        # [tokens, hidden], 32-bit
        previous = torch.where(first[:, None], carried, before)
        if write:
            last = (ctx.request_start[1:] - 1).long()
            cache.state.index_copy_(0, cache.slots.long(), x.float()[last])
        return self.ops.linear((x.float() + previous).to(x.dtype), self.mix)


def describe_shift(config: ToyConfig) -> ModelSpec:
    hidden = config.hidden_size
    norm = lambda prefix: PartSpec("rmsnorm", {"size": hidden, "eps": config.eps}, prefix)
    swiglu = PartSpec("swiglu", {"hidden": hidden, "width": config.width}, "ffn.")
    shift = PartSpec("toy_shift", {"hidden": hidden}, "shift.")
    conv = PartSpec("short_conv", {"hidden": hidden, "taps": 3, "bias": False}, "conv.")
    layers = tuple(LayerSpec(f"layers.{i}.", PartSpec("prenorm"), mixer, norm("norm1."), swiglu,
                             norm("norm2.")) for i, mixer in enumerate((shift, conv, shift)))
    return ModelSpec(architecture="toy-shift", vocab_size=config.vocab_size, hidden_size=hidden,
                     embedding="embed.weight", layers=layers,
                     order=tuple(LayerCall(i) for i in range(3)),
                     final_norm=norm("final_norm."), head=None, max_positions=4096)


def plain_shift(w, cfg: ToyConfig, ids):
    x = w["embed.weight"][torch.tensor(ids)]
    for layer in range(3):
        p = f"layers.{layer}."
        n = rms_norm(x, w[p + "norm1.weight"], cfg.eps)
        if layer == 1:
            bcx = n @ w[p + "conv.in_proj.weight"].T
            b, c, xs = bcx.chunk(3, dim=-1)
            g = torch.cat([torch.zeros(2, cfg.hidden_size), b * xs])
            kernel = w[p + "conv.conv"]
            y = sum(kernel[:, k] * g[k:k + len(ids)] for k in range(3))
            mixed = (c * y) @ w[p + "conv.out_proj.weight"].T
        else:
            previous = torch.cat([torch.zeros(1, cfg.hidden_size), n[:-1]])
            mixed = (n + previous) @ w[p + "shift.mix.weight"].T
        h = x + mixed
        n = rms_norm(h, w[p + "norm2.weight"], cfg.eps)
        gate, up = n @ w[p + "ffn.w1.weight"].T, n @ w[p + "ffn.w3.weight"].T
        x = h + (torch.nn.functional.silu(gate) * up) @ w[p + "ffn.w2.weight"].T
    return rms_norm(x, w["final_norm.weight"], cfg.eps) @ w["embed.weight"].T


def describe(config: ToyConfig) -> ModelSpec:
    hidden = config.hidden_size
    norm = lambda prefix: PartSpec("rmsnorm", {"size": hidden, "eps": config.eps}, prefix)
    swiglu = PartSpec("swiglu", {"hidden": hidden, "width": config.width}, "ffn.")
    rope = PartSpec("rope", {"theta": 1000.0, "rotary_dim": hidden // config.heads})
    decay = PartSpec("toy_decay", {"hidden": hidden}, "decay.")
    attention = PartSpec("attention", {"hidden": hidden, "heads": config.heads,
                                       "kv_heads": config.kv_heads,
                                       "head_dim": hidden // config.heads, "qk_norm_eps": None,
                                       "position": rope, "window": None, "scale": None}, "attn.")
    layers = tuple(LayerSpec(f"layers.{i}.", PartSpec("prenorm"), mixer, norm("norm1."), swiglu,
                             norm("norm2.")) for i, mixer in enumerate((decay, attention)))
    # layer 0 runs twice (each call with a state of its own); the last call runs layer 1 again
    # but reads the keys and values that the second call wrote, writing none itself
    order = (LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache=1, writes_cache=False))
    return ModelSpec(architecture="toy-decay", vocab_size=config.vocab_size, hidden_size=hidden,
                     embedding="embed.weight", layers=layers, order=order,
                     final_norm=norm("final_norm."), head="head.weight", max_positions=4096)


def plain_toy(w, cfg: ToyConfig, ids):
    """The same model over a whole sequence, written out plainly."""
    hd = cfg.hidden_size // cfg.heads
    x = w["embed.weight"][torch.tensor(ids)]

    def ffn(n, p):
        gate, up = n @ w[p + "ffn.w1.weight"].T, n @ w[p + "ffn.w3.weight"].T
        return (torch.nn.functional.silu(gate) * up) @ w[p + "ffn.w2.weight"].T

    def decay(n, p):
        rate = torch.sigmoid(w[p + "decay.decay"] * 50)
        state, rows = torch.zeros(cfg.hidden_size), []
        for row in n:
            state = rate * state + (1 - rate) * row
            rows.append(state)
        return torch.stack(rows) @ w[p + "decay.mix.weight"].T

    def project(n, p):
        tokens = n.shape[0]
        angles = rope_angles(torch.arange(tokens), hd, 1000.0)
        q = apply_rope((n @ w[p + "attn.q_proj.weight"].T).view(tokens, cfg.heads, hd), angles)
        k = apply_rope((n @ w[p + "attn.k_proj.weight"].T).view(tokens, cfg.kv_heads, hd), angles)
        v = (n @ w[p + "attn.v_proj.weight"].T).view(tokens, cfg.kv_heads, hd)
        return q, k, v

    def attend(q, k, v, p):
        tokens = q.shape[0]
        group = cfg.heads // cfg.kv_heads
        scores = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(group, 1)) * hd ** -0.5
        mask = torch.arange(tokens)[None, :] <= torch.arange(tokens)[:, None]
        scores = scores.masked_fill(~mask[None], float("-inf"))
        out = torch.einsum("hqk,khd->qhd", torch.softmax(scores, -1), v.repeat_interleave(group, 1))
        return out.reshape(tokens, -1) @ w[p + "attn.out_proj.weight"].T

    kept = None
    for call, layer in enumerate((0, 1, 0, 1)):
        p = f"layers.{layer}."
        n = rms_norm(x, w[p + "norm1.weight"], cfg.eps)
        if layer == 0:
            mixed = decay(n, p)
        else:
            q, k, v = project(n, p)
            if call == 1:
                kept = (k, v)
            mixed = attend(q, *kept, p)         # the last call reads the second call's keys
        h = x + mixed
        x = h + ffn(rms_norm(h, w[p + "norm2.weight"], cfg.eps), p)
    return rms_norm(x, w["final_norm.weight"], cfg.eps) @ w["head.weight"].T


@pytest.fixture()
def toy_registered():
    MIXERS.register("toy_decay", DecayMixer)
    register_architecture(Architecture("toy-decay", ToyConfig, describe))
    yield
    unregister_architecture("toy-decay")
    MIXERS.unregister("toy_decay")


def run_toy(tmp_path, device, dtype, ops):
    cfg = ToyConfig()
    folder = write_random_model(tmp_path / "toy", cfg.to_dict(), seed=5, dtype=torch.float32)
    assert json.loads((folder / "config.json").read_text())["model_type"] == "toy-decay"
    loaded = load_model(folder, dtype, device, ops=ops)
    model = loaded.model
    assert sorted(model.cache_needs) == [0, 1, 2]            # the fourth call has no entry
    cache = CacheManager(model.cache_needs, page_size=8, capacity_tokens=128, max_requests=3,
                         dtype=model.runtime.dtype, device=device)
    assert len(cache.states) == 1 and cache.states[0].storage.dtype == torch.float32
    runner = Runner(model, cache)
    from safetensors.torch import load_file
    weights = {k: v.float() for k, v in load_file(str(folder / "model.safetensors")).items()}
    requests = prompts(cfg.vocab_size, (23, 40), seed=1)
    steps = [([(0, part)], []) for part in cut(requests[0], (5, 2, 9))]
    steps += [([(1, requests[1][:30])], [])]
    steps += [([(1, [t])], []) for t in requests[1][30:]]
    # the two requests interleaved: portions of one beside tokens of the other
    mixed = []
    for i in range(max(len(steps), 1)):
        mixed.append(steps[i])
    got = replay(runner, cache, mixed)
    for i, tokens in enumerate(requests):
        assert_close(got[i], plain_toy(weights, cfg, tokens), model.runtime.dtype, f"toy {i}")


def test_toy_architecture_on_the_cpu(tmp_path, toy_registered):
    from plain_ops import PlainOps
    run_toy(tmp_path, "cpu", torch.float32, PlainOps())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_architecture_on_the_gpu(tmp_path, toy_registered, dtype):
    run_toy(tmp_path, "cuda:0", dtype, None)


@pytest.fixture()
def shift_registered():
    MIXERS.register("toy_shift", ShiftMixer)
    register_architecture(Architecture("toy-shift", ToyConfig, describe_shift))
    yield
    unregister_architecture("toy-shift")
    MIXERS.unregister("toy_shift")


def run_shift(tmp_path, device, dtype, ops):
    """Steps of two requests whose shape repeats with other splits of the tokens (24 + 17, then
    30 + 11, 17 + 24 ...) and decode steps: on the GPU they are captured and replayed."""
    import warnings

    cfg = ToyConfig(model_type="toy-shift")
    folder = write_random_model(tmp_path / "shift", cfg.to_dict(), seed=9, dtype=torch.float32)
    loaded = load_model(folder, dtype, device, ops=ops)
    model = loaded.model
    assert model.capturable
    cache = CacheManager(model.cache_needs, page_size=8, capacity_tokens=1024, max_requests=4,
                         dtype=model.runtime.dtype, device=device)
    runner = Runner(model, cache)
    from safetensors.torch import load_file
    weights = {k: v.float() for k, v in load_file(str(folder / "model.safetensors")).items()}
    a, b = prompts(cfg.vocab_size, (160, 140), seed=2)
    splits = [(24, 17), (24, 17), (24, 17), (30, 11), (17, 24), (1, 40), (39, 2)]
    steps, at_a, at_b = [], 0, 0
    for size_a, size_b in splits:
        steps.append(([("a", a[at_a:at_a + size_a]), ("b", b[at_b:at_b + size_b])], []))
        at_a, at_b = at_a + size_a, at_b + size_b
    while at_a < len(a) or at_b < len(b):                     # the rest token by token
        entries = []
        if at_a < len(a):
            entries.append(("a", [a[at_a]]))
            at_a += 1
        if at_b < len(b):
            entries.append(("b", [b[at_b]]))
            at_b += 1
        steps.append((entries, []))
    with warnings.catch_warnings():
        warnings.simplefilter("error")                         # no capture warning either
        got = replay(runner, cache, steps)
    assert_close(got["a"], plain_shift(weights, cfg, a), model.runtime.dtype, "shift a")
    assert_close(got["b"], plain_shift(weights, cfg, b), model.runtime.dtype, "shift b")
    return runner


def test_capturable_toy_on_the_cpu(tmp_path, shift_registered):
    from plain_ops import PlainOps
    run_shift(tmp_path, "cpu", torch.float32, PlainOps())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_capturable_toy_is_replayed_from_graphs(tmp_path, shift_registered, dtype):
    runner = run_shift(tmp_path, "cuda:0", dtype, None)
    # the 41-token shape was met seven times (captured at its second occurrence, so replayed six
    # times, four of them with another split), the decode shape a dozen times
    assert runner.graph_replays >= 6 + 8


@pytest.mark.gpu
def test_toys_that_cannot_be_captured_run_eagerly(tmp_path, toy_registered):
    """A model with a part that says ``capturable = False`` is never captured: no graph, no
    warning; and a part that reads host values although it claims to be capturable is told."""
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("error")
        run_toy(tmp_path, "cuda:0", torch.float32, None)
    DecayMixer.capturable = True
    try:
        with pytest.raises(RuntimeError, match="capturable"):
            run_toy(tmp_path / "again", "cuda:0", torch.float32, None)
    finally:
        DecayMixer.capturable = False
        torch.cuda.synchronize()
