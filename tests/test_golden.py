"""This repository's configuration, weight names, convolution state, paged attention, rotary
encoding and sampling rule against outputs of the reference's own code (tests/golden/reference_pieces.json, written by
tests/golden/make_golden.py from the parts of the reference that import without MLX)."""

import json
from pathlib import Path

import pytest
import torch

from mlx_one_b200.config import ConfigError, Lfm2Config
from mlx_one_b200.architectures.lfm2 import describe
from mlx_one_b200.parts.model import expected_tensors
from plain_lfm2 import (apply_rope, causal_attention, feed_forward_width, read_config,
                        rope_angles, sample_token)
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


def test_paged_attention_equals_the_reference_oracle():
    """The reference's NumPy paged attention (src/mlx_one/engine/paged_attention.py:209-246) on
    two requests with shuffled pages: the plain kernel restatement reads the same pool through a
    block table, and the plain model's whole-sequence attention sees the same keys in order.
    Pins the mapping of query heads to key heads, the causal bound and the scale."""
    from plain_ops import PlainOps
    from mlx_one_b200.parts.base import PagedKeyValues, PagedView, StepContext

    golden = GOLDEN["paged_attention"]
    heads, kv_heads, head_dim, page = (golden[k] for k in ("heads", "kv_heads", "head_dim", "page"))
    pool = torch.tensor(golden["pool"])                        # [2, pages, kv_heads, page, hd]
    queries = torch.tensor(golden["queries"])                  # [requests, heads, 3, hd]
    want = torch.tensor(golden["output"])
    width = max(len(t) for t in golden["tables"])
    table = torch.tensor([t + [-1] * (width - len(t)) for t in golden["tables"]], dtype=torch.int32)
    as_int = lambda v: torch.tensor(v, dtype=torch.int32)
    positions, owner, rows = [], [], []
    for r, count in enumerate(golden["widths"]):
        for i in range(count):
            positions.append(golden["positions"][r][i])
            owner.append(r)
            rows.append((r, i))
    q = torch.stack([queries[r, :, i] for r, i in rows])        # [tokens, heads, hd]
    starts = [0, golden["widths"][0], sum(golden["widths"])]
    ctx = StepContext(tokens=len(rows), requests=2, token_ids=as_int([0] * len(rows)),
                      positions=as_int(positions), token_request=as_int(owner),
                      request_start=as_int(starts),
                      history=as_int([golden["positions"][0][0], golden["positions"][1][0]]),
                      max_portion=3, max_context=max(golden["lengths"]))
    view = PagedView(pool, table, page, PagedKeyValues(kv_heads, head_dim))
    got = PlainOps().paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                     scale=golden["scale"], window=None, ctx=ctx, view=view)
    for t, (r, i) in enumerate(rows):
        torch.testing.assert_close(got[t].view(heads, head_dim), want[r, :, i], atol=1e-5, rtol=1e-5)
    # rows of request 1 that the oracle was not asked for stay zero (its widths say one query)
    assert torch.all(want[1, :, 1:] == 0)
    # the plain model's attention over request 0's keys in their logical order
    length = golden["lengths"][0]
    ordered = pool[:, golden["tables"][0]].permute(0, 1, 3, 2, 4).reshape(2, -1, kv_heads, head_dim)
    full_q = torch.zeros(length, heads, head_dim)
    for i, position in enumerate(golden["positions"][0]):
        full_q[position] = queries[0, :, i]
    whole = causal_attention(full_q, ordered[0, :length], ordered[1, :length])
    for i, position in enumerate(golden["positions"][0]):
        torch.testing.assert_close(whole[position], want[0, :, i], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("case", range(len(GOLDEN["rope"])))
def test_rotary_encoding_equals_the_reference(case):
    """The reference's apply_rope with explicit position_ids
    (src/mlx_one/models/shared/transformer.py:27-29, 50-51, 67-72, 88-90) against the plain
    implementation's angles and rotation, and against the engine's table of inverse
    frequencies."""
    from mlx_one_b200.parts.base import Runtime
    from mlx_one_b200.parts.positions import RotaryEncoding
    from mlx_one_b200.parts.spec import PartSpec

    golden = GOLDEN["rope"][case]
    value = torch.tensor(golden["value"])[0].permute(1, 0, 2)          # [tokens, heads, hd]
    want = torch.tensor(golden["rotated"])[0].permute(1, 0, 2)
    angles = rope_angles(torch.tensor(golden["positions"]), golden["head_dim"], golden["theta"])
    torch.testing.assert_close(apply_rope(value, angles), want, atol=2e-6, rtol=2e-6)
    part = RotaryEncoding(PartSpec("rope", {"theta": golden["theta"],
                                            "rotary_dim": golden["head_dim"]}), {},
                          Runtime(torch.float32, torch.device("cpu"), None))
    inv_freq, rotary_dim = part.rotary_table()
    assert rotary_dim == golden["head_dim"]
    engine_angles = torch.tensor(golden["positions"], dtype=torch.float32)[:, None] * inv_freq[None]
    torch.testing.assert_close(apply_rope(value, engine_angles), want, atol=2e-6, rtol=2e-6)


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
