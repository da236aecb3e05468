"""This repository's configuration, weight names, convolution state and sampling rule against
outputs of the reference's own code (tests/golden/reference_pieces.json, written by
tests/golden/make_golden.py from the parts of the reference that import without MLX)."""

import json
from pathlib import Path

import pytest
import torch

from mlx_one_b200.config import ConfigError, Lfm2Config
from mlx_one_b200.architectures.lfm2 import describe
from mlx_one_b200.parts.model import expected_tensors
from plain_lfm2 import feed_forward_width, read_config, sample_token
from plain_ops import kept_set
from tiny_models import TINY_A, TINY_B, TINY_C

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_pieces.json").read_text())
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "defaults": {"model_type": "lfm2"},
           "idxs": {"model_type": "lfm2", "num_hidden_layers": 6, "full_attn_idxs": [1, 4]}}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_derivations_equal_the_reference(name, tmp_path):
    want = GOLDEN["config"][name]
    cfg = Lfm2Config.from_dict(CONFIGS[name])
    assert cfg.adjusted_intermediate_size == want["intermediate"]
    assert list(cfg.layer_types) == want["layer_types"]
    assert list(cfg.full_attn_idxs) == want["full_attn_idxs"]
    assert cfg.rope_theta == want["rope_theta"]
    # the plain implementation reads config.json by itself and must agree too
    (tmp_path / "config.json").write_text(json.dumps(CONFIGS[name]))
    plain = read_config(tmp_path)
    assert feed_forward_width(plain) == want["intermediate"]
    assert plain["layer_types"] == want["layer_types"]


@pytest.mark.parametrize("name", ["A", "B", "C", "1.2B"])
def test_tensor_names_and_shapes_equal_the_reference_contract(name):
    data = CONFIGS.get(name)
    if data is None:
        import bench
        data = bench.LFM2_1_2B
    want = {k: tuple(v) for k, v in GOLDEN["config"][name]["tensors"].items()}
    got = {k: tuple(v.shape) for k, v in expected_tensors(describe(Lfm2Config.from_dict(data))).items()}
    assert got == want


def test_rejections_equal_the_reference():
    cases = {
        "odd_head": {"hidden_size": 30, "num_attention_heads": 2, "num_key_value_heads": 2},
        "heads": {"hidden_size": 64, "num_attention_heads": 3},
        "groups": {"num_attention_heads": 16, "num_key_value_heads": 5},
        "layer_count": {"num_hidden_layers": 3, "layer_types": ["conv"]},
        "layer_kind": {"num_hidden_layers": 1, "layer_types": ["mamba"]},
        "no_attention": {"num_hidden_layers": 2, "layer_types": ["conv", "conv"]},
        "window": {"num_hidden_layers": 1, "layer_types": ["sliding_attention"]},
        "swiglu": {"block_use_swiglu": False},
        "rope": {"rope_parameters": {"rope_type": "llama3"}},
        "eps": {"norm_eps": 0},
    }
    for name, data in cases.items():
        assert GOLDEN["rejected"][name] is not None
        with pytest.raises(ConfigError):
            Lfm2Config.from_dict({"model_type": "lfm2", **data})
    with pytest.raises(ConfigError):
        Lfm2Config.from_dict({"model_type": "llama"})


def test_convolution_state_equals_the_reference_cache():
    """The window that the reference's ConvCache hands to the convolution for every portion
    (src/mlx_one/core/cache.py:476-491) equals what the plain kernel restatement keeps."""
    from plain_ops import PlainOps
    from mlx_one_b200.parts.base import FixedState, StateView, StepContext

    golden = GOLDEN["conv_cache"]
    taps = golden["taps"]
    values = torch.tensor(golden["values"])[0]                 # [tokens, channels] = g
    channels = values.shape[1]
    state = torch.zeros(1, taps - 1, channels)
    ops = PlainOps()
    at = 0
    # a kernel of ones in tap k picks g[t - (taps-1) + k]; with B = 1, C = 1, x = g
    for cut, window in zip(golden["cuts"], golden["windows"]):
        part = values[at:at + cut]
        window = torch.tensor(window)[0]                       # [taps-1 + cut, channels]
        bcx = torch.cat((torch.ones_like(part), torch.ones_like(part), part), dim=1)
        as_int = lambda v: torch.tensor(v, dtype=torch.int32)
        ctx = StepContext(tokens=cut, requests=1, token_ids=as_int([0] * cut),
                          positions=as_int(list(range(at, at + cut))),
                          token_request=as_int([0] * cut), request_start=as_int([0, cut]),
                          history=as_int([at]), max_portion=cut, max_context=at + cut)
        for k in range(taps):
            kernel = torch.zeros(channels, taps)
            kernel[:, k] = 1
            view = StateView(state.clone(), as_int([0]), FixedState((taps - 1, channels)))
            got = ops.short_conv(bcx, kernel=kernel, bias=None, taps=taps, ctx=ctx, view=view,
                                 write=False)
            torch.testing.assert_close(got, window[k:k + cut])
        view = StateView(state, as_int([0]), FixedState((taps - 1, channels)))
        ops.short_conv(bcx, kernel=torch.zeros(channels, taps), bias=None, taps=taps, ctx=ctx,
                       view=view, write=True)
        at += cut


@pytest.mark.parametrize("case", range(len(GOLDEN["sampling"])))
def test_sampling_rule_equals_the_reference(case):
    golden = GOLDEN["sampling"][case]
    p = torch.tensor(golden["probabilities"])
    kept = set(kept_set(p, golden["top_k"] or 0, golden["top_p"]).tolist())
    # the golden set holds every token that one of 2000 evenly spaced draws returned, so it
    # may lack kept tokens whose share of the kept mass is below 1/2000, and nothing else
    assert set(golden["kept"]) <= kept
    mass = float(p[sorted(kept)].double().sum())
    for token in kept - set(golden["kept"]):
        assert float(p[token]) / mass < 1 / 2000
    # the plain restatement of the whole rule, fed Python's own random numbers
    import random
    for seed, want in enumerate(golden["python_random_picks"]):
        uniform = random.Random(seed).random()
        got = sample_token(torch.log(p), 1.0, golden["top_k"], golden["top_p"], uniform)
        assert got == want
