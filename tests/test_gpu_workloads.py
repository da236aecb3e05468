"""Workloads on the GPU that the small equality tests do not reach: a control that shows that
the comparison sees a wrong page, a model with the layer sizes of LFM2-1.2B through all four
cuts, the sampled mixed workload of five requests, and small twins of the benchmark's
continuous-batching and long-context cases."""

import pytest
import torch

from plain_lfm2 import PlainModel, counter_uniform
from plain_ops import kept_set
from tiny_models import (CONFIGS, assert_close, cut, make_model_dir, mixed_schedule, prompts,
                         replay, tolerance)

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def runner_for(folder, dtype, page_size, capacity, max_requests=8):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner

    loaded = load_model(folder, dtype, "cuda:0")
    cache = CacheManager(loaded.model.cache_needs, page_size=page_size, capacity_tokens=capacity,
                         max_requests=max_requests, dtype=dtype, device="cuda:0")
    return Runner(loaded.model, cache), cache


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: make_model_dir(name, root) for name in CONFIGS}


# ----------------------------------------------------------------------- a control


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_a_wrong_page_in_one_layer_is_seen(folders, name, dtype):
    """The comparison with the plain model must be able to fail: after a prompt has been run
    (and found equal), one page of ONE attention layer's keys and values is overwritten with
    another live page's contents, and the next decoded token's logits must be outside the
    tolerance. (Wrong data only: every address stays inside the storage.)"""
    config, _, page = CONFIGS[name]
    plain = PlainModel(folders[name])
    runner, cache = runner_for(folders[name], dtype, page, 256)
    (tokens,) = prompts(config["vocab_size"], (3 * page + 2,), seed=12)
    want = plain.logits(tokens)
    got = replay(runner, cache, [([("r", tokens[:-1])], [])])["r"]
    assert_close(got, want[:-1], dtype, f"{name} prompt")
    number, group = next((g, group) for g, group in enumerate(cache.paged)
                         if group.need.window is None)
    table = cache.get("r").tables[number]
    first, second = table[0], table[1]
    assert first >= 0 and second >= 0 and first != second
    layer = len(group.entries) - 1                      # the group's last layer
    group.storage[layer, :, first] = group.storage[layer, :, second].clone()
    spoilt = replay(runner, cache, [([("r", tokens[-1:])], ["r"])])["r"]
    with pytest.raises(AssertionError, match="logits differ"):
        assert_close(spoilt, want[-1:], dtype, f"{name} after a page was overwritten")


# ----------------------------------------------------------------------- real layer sizes

LAYERS_OF_1_2B = dict(
    model_type="lfm2", num_hidden_layers=3, layer_types=["conv", "full_attention", "conv"],
    hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
    block_auto_adjust_ff_dim=True, block_ff_dim=12288, block_multiple_of=256,
    block_ffn_dim_multiplier=1.0, vocab_size=65536, rope_theta=1000000.0, conv_L_cache=3,
    conv_bias=False, tie_embedding=True, norm_eps=1e-5, max_position_embeddings=128000)


@pytest.fixture(scope="module")
def real_size(tmp_path_factory):
    """Three layers with the sizes of LFM2-1.2B (hidden 2048, 32 heads over 8 key heads of 64,
    feed-forward 8192, vocabulary 65536), the plain model's logits for six requests."""
    from mlx_one_b200.weights import write_random_model

    folder = write_random_model(tmp_path_factory.mktemp("real") / "model", LAYERS_OF_1_2B, seed=4,
                                dtype=torch.bfloat16)
    plain = PlainModel(folder)
    requests = dict(enumerate(prompts(65536, (200, 90, 47, 130, 60, 150), seed=6)))
    return folder, requests, {i: plain.logits(t) for i, t in requests.items()}


@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_sizes_of_the_1_2b_model_through_every_cut(real_size, dtype):
    """What only real sizes reach inside the engine: the skinny product at K = 8192, SwiGLU
    tiles over 16384 columns, the 65536-row output product with its 32-bit store, 32 heads over
    8 key heads at head size 64 in both attention kernels, the in_proj + conv epilogue at
    hidden 2048, the tcgen05 products on whole prompts."""
    folder, requests, want = real_size
    capacity = 3 * 208
    runner, cache = runner_for(folder, dtype, 16, capacity, max_requests=3)
    tokens = requests[0]
    for forced in (False, True):                       # the dispatch rule's choice, then tcgen05 always
        runner.ops.tcgen05_always = forced
        try:
            got = replay(runner, cache, [([("w", tokens)], ["w"])])["w"]
        finally:
            runner.ops.tcgen05_always = False
        assert_close(got, want[0], dtype, f"whole, tcgen05 forced: {forced}")
    steps = [([("d", tokens[:168])], [])] + [([("d", [t])], []) for t in tokens[168:]]
    steps[-1] = (steps[-1][0], ["d"])
    assert_close(replay(runner, cache, steps)["d"], want[0], dtype, "last 32 one by one")
    for sizes in ((7, 2, 13, 3, 2, 5), (33, 1, 31, 16, 9)):
        steps = [([("p", part)], []) for part in cut(tokens, sizes)]
        steps[-1] = (steps[-1][0], ["p"])
        assert_close(replay(runner, cache, steps)["p"], want[0], dtype, f"portions {sizes}")
    # three live requests at a time in a pool that is smaller than all requests together, so
    # later requests get pages that earlier ones gave back
    assert sum(len(t) for t in requests.values()) > capacity
    got = replay(runner, cache, mixed_schedule(requests, live_limit=3))
    for request_id in requests:
        assert_close(got[request_id], want[request_id], dtype, f"mixed request {request_id}")
    assert not cache.requests()


# ----------------------------------------------------------------------- sampled workload


def token_order_draw(logits, temperature, top_k, top_p, seed, step):
    """The engine's documented draw on plain logits: the reference's kept set
    (src/mlx_one/text/sampling.py:56-81), walked in token order with the counter-based
    number of (seed, step). Returns (token, how far the number lies from the nearest edge of
    the chosen token's interval, as a fraction of the kept mass)."""
    p = torch.softmax(logits.double() / temperature, dim=-1)
    kept = kept_set(p, top_k or 0, top_p)
    weights = torch.zeros_like(p)
    weights[kept] = p[kept]
    running = torch.cumsum(weights, dim=0)
    mass = float(weights.sum())
    target = counter_uniform(seed, step) * mass
    hit = torch.nonzero((running >= target) & (weights > 0))
    token = int(hit[0]) if len(hit) else int(kept.max())
    upper = float(running[token])
    lower = upper - float(weights[token])
    return token, min(target - lower, upper - target) / mass


@pytest.mark.parametrize("pipeline", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
def test_five_sampled_requests_in_portions_of_16(folders, dtype, pipeline):
    """Tiny model B's workload: five requests of 1, 9, 33, 64 and 100 prompt tokens, prompt
    portions of 16 tokens beside ongoing decodes, 24 tokens each at temperature 0.8 with a seed
    per request, pages of 8. Every drawn token equals the plain draw on the plain model's
    logits. In bfloat16 a token may differ only where the random number lies within the
    logits' tolerance of an edge of the cumulative distribution; that request is compared no
    further."""
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions

    config, _, page = CONFIGS["B"]
    plain = PlainModel(folders["B"])
    engine = Engine(folders["B"], execution_dtype=dtype, device="cuda:0",
                    cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=1024),
                    batching_config=BatchingConfig(max_sequences=5, queue_size=8,
                                                   prefill_chunk_size=16, max_prefill_tokens=32,
                                                   max_scheduled_tokens=40,
                                                   pipeline_decode=pipeline))
    requests = prompts(config["vocab_size"], (1, 9, 33, 64, 100), seed=14)
    options = [TextGenerationOptions(max_tokens=24, temperature=0.8, seed=100 + i)
               for i in range(5)]
    results = engine.generate_batch_ids(requests, options)
    traces = engine.step_traces()
    assert any(t["phase"] == "mixed" for t in traces)            # portions beside decodes
    assert max(t["prompt_tokens"] for t in traces) <= 32
    compared = 0
    for i, (prompt, result) in enumerate(zip(requests, results)):
        assert result.generation_tokens == 24 and result.finish_reason == "length"
        ids = list(prompt)
        for step, token in enumerate(result.token_ids):
            logits = plain.logits(ids)[-1]
            expected, margin = token_order_draw(logits, 0.8, None, 1.0, 100 + i, step)
            if token != expected:
                atol, rtol = tolerance(dtype, logits)
                slack = 2 * (atol + rtol * float(logits.abs().max())) / 0.8
                assert dtype == torch.bfloat16 and margin < slack, (
                    f"request {i} token {step}: drew {token}, the plain draw is {expected} "
                    f"(margin {margin:.2e})")
                break
            compared += 1
            ids.append(token)
    assert compared >= (120 if dtype == torch.float32 else 60)
    engine.model.ops.check_errors()
    engine.close()
    assert not engine.cache.requests()
