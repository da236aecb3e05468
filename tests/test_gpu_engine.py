"""The engine on the GPU against the plain implementation: whole requests, the last tokens
one by one, portions of changing size, and mixed batches with pages used again."""

import pytest
import torch

from plain_lfm2 import PlainModel
from tiny_models import (CONFIGS, assert_close, cut, make_model_dir, mixed_schedule, prompts,
                         replay)

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: make_model_dir(name, root) for name in CONFIGS}


@pytest.fixture(scope="module")
def plain(folders):
    return {name: PlainModel(folder) for name, folder in folders.items()}


def engine(folder, dtype, page_size, capacity, max_requests=8):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner

    loaded = load_model(folder, dtype, "cuda:0")
    cache = CacheManager(loaded.model.cache_needs, page_size=page_size, capacity_tokens=capacity,
                         max_requests=max_requests, dtype=dtype, device="cuda:0")
    return Runner(loaded.model, cache), cache


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_requests(folders, plain, name, dtype):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 256)
    for i, tokens in enumerate(prompts(config["vocab_size"], (7, 13, 21, 100, 1))):
        got = replay(runner, cache, [([(i, tokens)], [i])])[i]
        assert_close(got, plain[name].logits(tokens), dtype, f"{name} whole request {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_last_tokens_one_by_one(folders, plain, name, dtype):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 256)
    (tokens,) = prompts(config["vocab_size"], (97,), seed=3)
    steps = [([("r", tokens[:65])], [])] + [([("r", [t])], []) for t in tokens[65:]]
    got = replay(runner, cache, steps)["r"]
    assert_close(got, plain[name].logits(tokens), dtype, f"{name} decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_changing_size(folders, plain, name, dtype):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 256)
    (tokens,) = prompts(config["vocab_size"], (131,), seed=4)
    for sizes in ((7, 2, 13, 3, 2, 5), (2,), (33, 1, 31)):
        steps = [([("r", part)], []) for part in cut(tokens, sizes)]
        steps[-1] = (steps[-1][0], ["r"])
        got = replay(runner, cache, steps)["r"]
        assert_close(got, plain[name].logits(tokens), dtype, f"{name} portions {sizes}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_page_reuse(folders, plain, name, dtype):
    """Up to four live requests, portions of some beside decoded tokens of others, in a pool
    so small that pages of finished requests are handed to later ones."""
    config, _, page = CONFIGS[name]
    lengths = (40, 64, 23, 50, 17, 61, 9, 33)
    requests = dict(enumerate(prompts(config["vocab_size"], lengths, seed=5)))
    capacity = 4 * 64
    runner, cache = engine(folders[name], dtype, page, capacity, max_requests=4)
    steps = mixed_schedule(requests)
    got = replay(runner, cache, steps)
    assert cache.stats().pages_low_water[0] < cache.stats().pages_total[0] // 2
    for request_id, tokens in requests.items():
        assert_close(got[request_id], plain[name].logits(tokens), dtype,
                     f"{name} mixed request {request_id}")
    assert not cache.requests()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_steps_of_a_repeated_shape_are_replayed(folders, plain, name, dtype):
    """Steps with portions whose shape comes back (two requests, 24 + 17 tokens, then a portion
    beside a decoded token) are captured as graphs at their third occurrence and replayed:
    different tokens, different pages, different histories, the same shape. The shape says
    how many tokens and requests a step has, not how the tokens are split between the requests:
    later pairs bring 30 + 11 and 11 + 7 tokens to the graphs captured on 24 + 17 and 17 + 1."""
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 512)
    requests = dict(enumerate(prompts(config["vocab_size"], [42, 35] * 6, seed=9)))
    for pair in range(6):
        a, b = requests[2 * pair], requests[2 * pair + 1]
        first, second = ((24, 17), (17, 1)) if pair < 3 or pair == 4 else ((30, 11), (11, 7))
        a1, b1 = first[0], first[1]
        a2, b2 = a1 + second[0], b1 + second[1]
        assert (a2, b2) == (41, 18)
        steps = [([(2 * pair, a[:a1]), (2 * pair + 1, b[:b1])], []),
                 ([(2 * pair, a[a1:a2]), (2 * pair + 1, b[b1:b2])], []),
                 ([(2 * pair, a[a2:]), (2 * pair + 1, b[b2:])], [2 * pair, 2 * pair + 1])]
        got = replay(runner, cache, steps)
        assert_close(got[2 * pair], plain[name].logits(a), dtype, f"{name} pair {pair} a")
        assert_close(got[2 * pair + 1], plain[name].logits(b), dtype, f"{name} pair {pair} b")
    assert runner.use_graphs and runner.graph_replays >= 9        # three shapes, pairs 2 to 5


@pytest.mark.parametrize("dtype", DTYPES)
def test_mid_size_model_with_long_portions(tmp_path, dtype):
    """Hidden size 512, head size 64, a feed-forward width that is no multiple of 64, and
    portions of 300+ tokens: the kernels for large steps (tcgen05 products with fused
    epilogues, the wide conv and q/k kernels, prefill attention over several tiles) run inside
    the engine, next to decode steps, against the plain implementation."""
    from tiny_models import ALL_CONFIGS
    config, _, page = ALL_CONFIGS["MID"]
    folder = make_model_dir("MID", tmp_path)
    model = PlainModel(folder)
    runner, cache = engine(folder, dtype, page, 2048, max_requests=4)
    runner.ops.tcgen05_always = True       # every product that can, also where the library is faster
    a, b = prompts(config["vocab_size"], (700, 330), seed=31)
    steps = [([("a", a[:384])], []), ([("a", a[384:690]), ("b", b[:300])], [])]
    steps += [([("a", [t]), ("b", [u])], []) for t, u in zip(a[690:], b[300:310])]
    steps += [([("b", b[310:])], ["a", "b"])]
    try:
        got = replay(runner, cache, steps)
    finally:
        runner.ops.tcgen05_always = False
    if dtype == torch.bfloat16:
        assert runner.ops.tcgen05_products
    assert_close(got["a"], model.logits(a), dtype, "mid a")
    assert_close(got["b"], model.logits(b), dtype, "mid b")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_of_thousands_of_tokens(folders, plain, dtype):
    """5000 tokens of the head-size-64 model in portions of up to 2048 tokens and a decoded tail:
    attention over hundreds of pages and dozens of key tiles, the window long past its first
    pages, and the pages that the window left given back while the request lives."""
    config, _, page = CONFIGS["D"]
    (tokens,) = prompts(config["vocab_size"], (5000,), seed=77)
    runner, cache = engine(folders["D"], dtype, page, 5056, max_requests=2)
    sizes = [2048, 1300, 1024, 600] + [1] * 28
    assert sum(sizes) == len(tokens)
    steps, at = [], 0
    for size in sizes:
        steps.append(([("long", tokens[at:at + size])], []))
        at += size
    steps[-1] = (steps[-1][0], ["long"])
    got = replay(runner, cache, steps)["long"]
    assert_close(got, plain["D"].logits(tokens), dtype, "long prompt")
