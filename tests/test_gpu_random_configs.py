"""Seeded random LFM2 configurations (head sizes in steps of 16 and some that are not, odd head
counts and groups, widths and vocabularies that are no power of two, kernel widths 1 to 5, with
and without biases, windows, tied and separate heads, page sizes 1 to 64) replayed through the
engine in mixed batches with few pages, against the plain implementation, in both dtypes."""

import random

import pytest
import torch

from plain_lfm2 import PlainModel
from tiny_models import assert_close, mixed_schedule, prompts, replay

pytestmark = pytest.mark.gpu


def random_config(seed):
    rng = random.Random(seed)
    head_dim = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 8, 24, 40])
    kv_heads = rng.choice([1, 2, 3])
    heads = kv_heads * rng.choice([1, 2, 3, 5])
    layers = rng.randint(2, 5)
    kinds = [rng.choice(["conv", "full_attention", "sliding_attention"]) for _ in range(layers)]
    kinds[rng.randrange(layers)] = "full_attention"
    config = dict(
        model_type="lfm2", num_hidden_layers=layers, layer_types=kinds,
        hidden_size=heads * head_dim, num_attention_heads=heads, num_key_value_heads=kv_heads,
        vocab_size=rng.choice([257, 512, 1000, 1531]), rope_theta=rng.choice([1e4, 1e6, 5e5]),
        conv_L_cache=rng.randint(1, 5), conv_bias=rng.random() < 0.5,
        tie_embedding=rng.random() < 0.5, norm_eps=rng.choice([1e-5, 1e-6, 3e-5]),
        sliding_window=rng.choice([5, 17, 32, 33, 64]))
    if rng.random() < 0.5:
        config.update(block_auto_adjust_ff_dim=False, block_ff_dim=rng.choice([100, 136, 333, 512]))
    else:
        config.update(block_auto_adjust_ff_dim=True, block_ff_dim=rng.choice([300, 511, 768]),
                      block_multiple_of=rng.choice([1, 8, 20, 64]),
                      block_ffn_dim_multiplier=rng.choice([1.0, 1.3, 0.7]))
    return config, rng.choice([1, 2, 4, 8, 16, 32, 64])


@pytest.mark.parametrize("seed", range(12))
def test_random_configuration(tmp_path, seed):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner
    from mlx_one_b200.weights import write_random_model

    config, page = random_config(seed)
    stored = torch.float32 if seed % 3 == 0 else torch.bfloat16     # some checkpoints are 32-bit
    folder = write_random_model(tmp_path / "model", config, seed, stored)
    plain = PlainModel(folder)
    lengths = (150, 40, 64, 23, 9, 70)
    requests = dict(enumerate(prompts(config["vocab_size"], lengths, seed=seed)))
    expected = {i: plain.logits(tokens) for i, tokens in requests.items()}
    for dtype in (torch.float32, torch.bfloat16):
        loaded = load_model(folder, dtype, "cuda:0")
        cache = CacheManager(loaded.model.cache_needs, page_size=page, capacity_tokens=384,
                             max_requests=4, dtype=dtype, device="cuda:0")
        runner = Runner(loaded.model, cache)
        # the longest request alone and whole (a large step), then all of them mixed
        whole = replay(runner, cache, [([("w", requests[0])], ["w"])])["w"]
        assert_close(whole, expected[0], dtype, f"seed {seed} {config} whole")
        got = replay(runner, cache, mixed_schedule(requests, decode_tail=12))
        for i in requests:
            assert_close(got[i], expected[i], dtype, f"seed {seed} {config} request {i}")
        assert not cache.requests()
