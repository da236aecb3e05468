"""The engine's bookkeeping on the CPU: the step function, block tables, slots, scheduler and
entry point run with the plain kernel restatements (tests/plain_ops.py) in the place of the
CUDA kernels, and are compared with the plain implementation. What these tests can find are
faults of batching and caching; the kernels themselves are tested on the GPU."""

import pytest
import torch

from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions
from mlx_one_b200.cache import CacheManager
from mlx_one_b200.engine.loading import load_model
from mlx_one_b200.engine.runner import Runner, StepEntry
from plain_lfm2 import PlainModel, counter_uniform, sample_token
from plain_ops import PlainOps, uniform
from tiny_models import (CONFIGS, assert_close, cut, make_model_dir, mixed_schedule, prompts,
                         replay)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name in CONFIGS:
        folder = make_model_dir(name, root, dtype=torch.float32)
        out[name] = (folder, load_model(folder, "float32", "cpu", ops=PlainOps()),
                     PlainModel(folder))
    return out


def runner_for(loaded, page, capacity, max_requests=8):
    cache = CacheManager(loaded.model.cache_needs, page_size=page, capacity_tokens=capacity,
                         max_requests=max_requests, dtype=torch.float32, device="cpu")
    return Runner(loaded.model, cache), cache


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_decode_and_portions(models, name):
    folder, loaded, plain = models[name]
    config, _, page = CONFIGS[name]
    runner, cache = runner_for(loaded, page, 256)
    (tokens,) = prompts(config["vocab_size"], (70,), seed=2)
    want = plain.logits(tokens)
    whole = replay(runner, cache, [([("w", tokens)], ["w"])])["w"]
    assert_close(whole, want, torch.float32, "whole")
    steps = [([("d", tokens[:38])], [])] + [([("d", [t])], []) for t in tokens[38:]]
    assert_close(replay(runner, cache, steps)["d"], want, torch.float32, "decode")
    cache.close("d")
    for sizes in ((7, 2, 13, 3, 2, 5), (2,)):
        steps = [([("p", part)], []) for part in cut(tokens, sizes)]
        steps[-1] = (steps[-1][0], ["p"])
        assert_close(replay(runner, cache, steps)["p"], want, torch.float32, f"portions {sizes}")


def test_a_step_that_wants_every_row_in_order_picks_none(models):
    """Single tokens that all want their logits (a decode step): the step function hands the
    output product every row as it is, without the row gather, and each request gets the logits
    of its whole sequence's last position."""
    folder, loaded, plain = models["A"]
    config, _, page = CONFIGS["A"]
    runner, cache = runner_for(loaded, page, 256)
    requests = prompts(config["vocab_size"], (9, 14, 5), seed=12)
    for i, tokens in enumerate(requests):
        cache.open(i)
        runner.step([StepEntry(i, tokens[:-1])])
    picked = []
    gather = loaded.model.ops.gather_rows
    loaded.model.ops.gather_rows = lambda *a, **k: (picked.append(1), gather(*a, **k))[1]
    try:
        every = runner.step([StepEntry(i, [tokens[-1]], (0,)) for i, tokens in enumerate(requests)])
        assert not picked
    finally:
        loaded.model.ops.gather_rows = gather
    for i, tokens in enumerate(requests):
        assert_close(every[i:i + 1], plain.logits(tokens)[-1:], torch.float32, f"request {i}")
        cache.close(i)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_reuse_pages(models, name):
    folder, loaded, plain = models[name]
    config, _, page = CONFIGS[name]
    requests = dict(enumerate(prompts(config["vocab_size"], (40, 64, 23, 50, 17, 61), seed=5)))
    runner, cache = runner_for(loaded, page, 4 * 64, max_requests=4)
    got = replay(runner, cache, mixed_schedule(requests))
    stats = cache.stats()
    assert stats.pages_low_water[0] < stats.pages_total[0] // 2          # pages were reused
    for request_id, tokens in requests.items():
        assert_close(got[request_id], plain.logits(tokens), torch.float32, f"request {request_id}")
    assert not cache.requests()


def test_step_refuses_bad_batches_before_touching_state(models):
    folder, loaded, plain = models["A"]
    runner, cache = runner_for(loaded, 4, 32)
    cache.open("a")
    cache.open("b")
    for bad in ([StepEntry("a", [1]), StepEntry("a", [2])], [StepEntry("a", [])],
                [StepEntry("a", [512])], [StepEntry("a", [1, 2], [2])],
                [StepEntry("unknown", [1])]):
        with pytest.raises((ValueError, RuntimeError)):
            runner.step(bad)
    from mlx_one_b200.cache import CacheCapacityError
    runner.step([StepEntry("a", list(range(20)))])
    with pytest.raises(CacheCapacityError):
        runner.step([StepEntry("b", list(range(20)))])          # 12 tokens of room are left
    assert cache.get("b").length == 0 and cache.get("a").length == 20
    cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_entry_point_greedy_and_seeded_sampling(models, name):
    folder, loaded, plain = models[name]
    config, _, page = CONFIGS[name]
    engine = Engine(loaded, cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=512),
                    batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=16,
                                                   max_scheduled_tokens=24))
    requests = prompts(config["vocab_size"], (1, 9, 33, 64), seed=8)
    results = engine.generate_batch_ids(requests, TextGenerationOptions(max_tokens=6))
    for prompt, result in zip(requests, results):
        assert list(result.token_ids) == plain.greedy(prompt, 6)
        assert result.finish_reason == "length" and result.prompt_tokens == len(prompt)
    # sampled tokens follow the documented draw and do not depend on the batch
    options = TextGenerationOptions(max_tokens=5, temperature=0.8, top_k=40, top_p=0.95, seed=3)
    alone = engine.generate_ids(requests[1], options).token_ids
    together = engine.generate_batch_ids(requests[:3], options)[1].token_ids
    assert alone == together
    ids = list(requests[1])
    for step, token in enumerate(alone):
        assert uniform(3, step) == counter_uniform(3, step)
        logits = plain.logits(ids)[-1]
        kept_draw = PlainOps().sample(logits[None], torch.tensor([0.8]), torch.tensor([40]),
                                      torch.tensor([0.95]), torch.tensor([3]),
                                      torch.tensor([step]))[0]
        assert int(kept_draw[0]) == token
        ids.append(token)
    streamed = [c.token_id for c in engine.stream_ids(requests[2], max_tokens=4)]
    assert streamed[:-1] == plain.greedy(requests[2], 4) and streamed[-1] is None
    stats = engine.runtime_stats()
    assert stats["running"] == 0 and stats["pages_free"] == stats["pages_total"]
    engine.close()


def test_end_token_stops_generation(models):
    folder, loaded, plain = models["A"]
    prompt = prompts(512, (12,), seed=1)[0]
    expected = plain.greedy(prompt, 3)
    import dataclasses
    spec = dataclasses.replace(loaded.spec, eos_token_ids=(expected[2],))
    patched = dataclasses.replace(loaded, spec=spec)
    engine = Engine(patched, cache_config=CacheConfig(block_size_tokens=4, capacity_tokens=128))
    result = engine.generate_ids(prompt, max_tokens=10)
    assert result.finish_reason == "stop" and list(result.token_ids) == expected[:expected.index(expected[2])]
    keep_going = engine.generate_ids(prompt, max_tokens=4, ignore_eos=True)
    assert keep_going.finish_reason == "length" and len(keep_going.token_ids) == 4


@pytest.mark.parametrize("pipeline", [True, False])
def test_pipelined_decode_gives_the_same_tokens(models, pipeline):
    """Requests of different lengths, one ending on an end-of-sequence token: launching a step
    before the last one is committed changes nothing but the number of steps run."""
    import dataclasses
    folder, loaded, plain = models["B"]
    requests = prompts(1000, (5, 9, 20), seed=13)
    lengths = (12, 3, 7)
    expected = [plain.greedy(p, n) for p, n in zip(requests, lengths)]
    eos = expected[0][5]                                  # request 0 stops at its sixth token
    cut = lambda tokens: tokens[:tokens.index(eos)] if eos in tokens else tokens
    spec = dataclasses.replace(loaded.spec, eos_token_ids=(eos,))
    engine = Engine(dataclasses.replace(loaded, spec=spec),
                    cache_config=CacheConfig(block_size_tokens=8, capacity_tokens=512),
                    batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=16,
                                                   max_scheduled_tokens=32,
                                                   pipeline_decode=pipeline))
    handles = [engine.submit_ids(p, max_tokens=n) for p, n in zip(requests, lengths)]
    engine.run()
    for handle, want in zip(handles, expected):
        result = handle.result()
        assert list(result.token_ids) == cut(want)
        assert result.finish_reason == ("stop" if eos in want else "length")
    stats = engine.runtime_stats()
    assert (stats["steps_ahead"] > 0) == pipeline
    assert stats["running"] == 0 and stats["pages_free"] == stats["pages_total"]
    engine.cache.check()


def test_coroutines_share_the_engine(models):
    """``async_generate_ids`` from several coroutines at once: every request is waited for on a
    thread of its own, the threads take turns at the loop, and each request gets the tokens it
    gets alone. A cancelled coroutine ends its request and gives its pages back."""
    import asyncio

    folder, loaded, plain = models["B"]
    config, _, page = CONFIGS["B"]
    engine = Engine(loaded, cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=512),
                    batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=16,
                                                   max_scheduled_tokens=24))
    requests = prompts(config["vocab_size"], (5, 21, 40, 9), seed=12)

    async def together():
        return await asyncio.gather(*(engine.async_generate_ids(p, max_tokens=7) for p in requests))

    for prompt, result in zip(requests, asyncio.run(together())):
        assert list(result.token_ids) == plain.greedy(prompt, 7)

    async def cancelled():
        long = asyncio.ensure_future(engine.async_generate_ids(requests[2], max_tokens=200))
        short = asyncio.ensure_future(engine.async_generate_ids(requests[0], max_tokens=3))
        await short
        long.cancel()
        with pytest.raises(asyncio.CancelledError):
            await long
        return short.result()

    short = asyncio.run(cancelled())
    assert list(short.token_ids) == plain.greedy(requests[0], 3)
    engine.run()
    stats = engine.runtime_stats()
    assert stats["running"] == 0 and stats["pages_free"] == stats["pages_total"]
    engine.close()


@pytest.mark.parametrize("pipeline", [True, False])
def test_a_timed_out_request_raises_and_the_others_finish(models, pipeline):
    """The clock passes a request's deadline while it decodes (also while steps are launched
    ahead): waiting for it raises RequestTimeoutError, the other request's tokens are what it
    gets alone, and every page comes back."""
    from mlx_one_b200.engine import RequestTimeoutError

    folder, loaded, plain = models["A"]
    config, _, page = CONFIGS["A"]
    engine = Engine(loaded, cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=512),
                    batching_config=BatchingConfig(max_sequences=2, timeout=50.0,
                                                   pipeline_decode=pipeline))
    now = [0.0]
    engine._scheduler.clock = lambda: now[0]
    slow_prompt, quick_prompt = prompts(config["vocab_size"], (9, 14), seed=21)
    slow = engine.submit_ids(slow_prompt, max_tokens=400, ignore_eos=True)
    for _ in range(6):
        engine.step()
    now[0] = 40.0
    quick = engine.submit_ids(quick_prompt, max_tokens=12, ignore_eos=True)
    for _ in range(5):
        engine.step()
    now[0] = 55.0                                   # past the first deadline, before the second
    assert list(quick.result().token_ids) == plain.greedy(quick_prompt, 12)
    with pytest.raises(RequestTimeoutError):
        slow.result()
    assert 0 < len(slow.request.output) < 400
    engine.run()
    stats = engine.runtime_stats()
    assert stats["running"] == 0 and stats["pages_free"] == stats["pages_total"]
    with pytest.raises(RequestTimeoutError):
        now[0] = 0.0
        stream = engine.stream_ids(slow_prompt, max_tokens=400, ignore_eos=True)
        for count, _ in enumerate(stream):
            if count == 3:
                now[0] = 1000.0
    engine.close()


@pytest.mark.parametrize("seed", range(12))
def test_random_load_on_the_entry_point(models, seed):
    """Requests that arrive while others run, with random lengths, budgets, portion sizes and
    numbers of sequences, a cache so small that some must wait, some cancelled on the way: every
    finished request has the tokens it gets alone, nothing is lost and every page comes back.
    In half of the runs a sixth of the vocabulary ends a sequence, so that requests end on a
    token that a step launched ahead has already been planned past."""
    import dataclasses
    import random

    rng = random.Random(seed)
    name = rng.choice(["A", "B", "C"])
    folder, loaded, plain = models[name]
    config, _, page = CONFIGS[name]
    ends = ()
    if seed >= 6:
        ends = tuple(rng.sample(range(config["vocab_size"]), config["vocab_size"] // 6))
        loaded = dataclasses.replace(loaded, spec=dataclasses.replace(loaded.spec,
                                                                      eos_token_ids=ends))
    budget = rng.choice([3, 8, 24, 64])
    engine = Engine(loaded,
                    cache_config=CacheConfig(block_size_tokens=page,
                                             capacity_tokens=rng.choice([96, 160, 512])),
                    batching_config=BatchingConfig(
                        max_sequences=rng.choice([1, 2, 3, 5]), queue_size=64,
                        prefill_chunk_size=rng.choice([2, 5, 16, 64]), max_scheduled_tokens=budget,
                        max_prefill_tokens=rng.choice([budget, max(budget // 2, 1)]),
                        pipeline_decode=rng.random() < 0.5))
    lengths = [rng.choice([1, 2, rng.randint(3, 20), rng.randint(20, 45)]) for _ in range(9)]
    waiting = list(zip(prompts(config["vocab_size"], lengths, seed=100 + seed),
                       [rng.randint(1, 9) for _ in lengths]))
    handles, cancelled = [], set()
    while waiting or engine._scheduler.has_work() or engine._inflight is not None:
        while waiting and rng.random() < 0.4:
            prompt, count = waiting.pop(0)
            handles.append((prompt, count, engine.submit_ids(prompt, max_tokens=count,
                                                             ignore_eos=not ends)))
        if handles and rng.random() < 0.05:
            index = rng.randrange(len(handles))
            if not handles[index][2].done():
                handles[index][2].cancel()
                cancelled.add(index)
        engine.step()
        engine.cache.check()
    assert len(handles) == len(lengths)
    for index, (prompt, count, handle) in enumerate(handles):
        result = handle.result()
        want = plain.greedy(prompt, count)
        ended = next((i for i, token in enumerate(want) if token in ends), None)
        if index in cancelled:
            assert list(result.token_ids) == want[:len(result.token_ids)]
            assert ended is None or len(result.token_ids) <= ended
        elif ended is not None:
            assert list(result.token_ids) == want[:ended] and result.finish_reason == "stop"
        else:
            assert list(result.token_ids) == want and result.finish_reason == "length"
    stats = engine.runtime_stats()
    assert stats["running"] == 0 and stats["waiting"] == 0
    assert stats["pages_free"] == stats["pages_total"]
    engine.close()


def test_every_step_leaves_a_record(models):
    """Per-step records as the reference's runners keep them: which requests, how many prompt
    and decode tokens, how many tokens were drawn, whether the step was launched ahead; the
    sink gets every record."""
    folder, loaded, plain = models["A"]
    config, _, page = CONFIGS["A"]
    seen = []
    engine = Engine(loaded, cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=256),
                    batching_config=BatchingConfig(max_sequences=2, prefill_chunk_size=8,
                                                   max_scheduled_tokens=16),
                    trace_sink=seen.append)
    first, second = prompts(config["vocab_size"], (19, 5), seed=4)
    results = engine.generate_batch_ids([first, second], TextGenerationOptions(max_tokens=4))
    records = engine.step_traces()
    assert records == seen and [r["step"] for r in records] == list(range(len(records)))
    assert sum(r["prompt_tokens"] for r in records) == len(first) + len(second)
    assert sum(r["draws"] for r in records) >= sum(len(r.token_ids) for r in results)
    assert records[0]["phase"] == "prefill" and records[0]["tokens"] <= 16
    assert any(r["phase"] == "mixed" for r in records)       # a decode beside a prompt portion
    assert records[-1]["phase"] == "decode" and records[-1]["prompt_tokens"] == 0
    # every step but the first is launched while the one before it is still in flight, steps
    # with prompt portions too
    assert all(r["launched_ahead"] for r in records[1:]) and not records[0]["launched_ahead"]
    assert any(r["launched_ahead"] and r["phase"] == "mixed" for r in records)
    for prompt, result in zip((first, second), results):
        assert list(result.token_ids) == plain.greedy(prompt, 4)
    assert all(r["duration_s"] >= 0 and r["batch_size"] == len(r["request_ids"]) for r in records)
    assert engine.runtime_stats()["steps_committed"] == len(records)


def test_hidden_states_can_be_watched_layer_by_layer(models):
    """``Model.observer`` sees the stream after the embedding and after every layer: the hidden
    states of a request cut into steps equal the plain implementation's, layer by layer."""
    import plain_lfm2

    folder, loaded, plain = models["C"]
    config, _, page = CONFIGS["C"]
    (tokens,) = prompts(config["vocab_size"], (23,), seed=17)
    runner, cache = runner_for(loaded, page, 64)
    seen = {}

    def watch(place, residual, delta):
        state = residual if delta is None else residual + delta.to(residual.dtype)
        seen.setdefault(place, []).append(state.clone())

    loaded.model.observer = watch
    try:
        replay(runner, cache, [([("r", tokens[:9])], []), ([("r", tokens[9:21])], []),
                               ([("r", tokens[21:22])], []), ([("r", tokens[22:])], ["r"])])
    finally:
        loaded.model.observer = None
    x = plain.w["model.embed_tokens.weight"][torch.tensor(tokens)]
    assert torch.equal(torch.cat(seen[-1]), x)
    for index in range(plain.cfg["num_hidden_layers"]):
        x = plain_lfm2.decoder_layer(x, plain.w, index, plain.cfg)
        torch.testing.assert_close(torch.cat(seen[index]), x, atol=1e-4, rtol=1e-4)


def test_shapes_are_rounded_up_with_fillers_that_have_tokens(models):
    """The rule by which a step's shape is rounded up for CUDA graphs: the leading single-token
    requests and the wanted rows to a multiple of 8, the other requests to a multiple of 2 and
    their tokens to a multiple of 64 (16 up to 128 tokens); a filler request has at least one
    token, filler tokens belong to a filler request, and a decode-only step stays decode-only
    (small ones stay as they are)."""
    folder, loaded, plain = models["A"]
    runner, cache = runner_for(loaded, 4, 64)
    for singles in (0, 1, 7, 8, 9, 63):
        for others in (1, 2, 3, 5):
            for other_tokens in list(range(others, others + 40)) + [others + 200, others + 511]:
                for wanted in (0, 1, singles + others):
                    more_s, more_o, more_t, more_w = runner._fill(singles, others, other_tokens,
                                                                  wanted)
                    assert (singles + more_s) % 8 == 0 and (wanted + more_w) % 8 == 0
                    assert (others + more_o) % 2 == 0
                    assert (other_tokens + more_t) % (64 if other_tokens > 128 else 16) == 0
                    assert more_t >= more_o >= 0 and (more_o > 0) == (more_t > 0)
                    assert more_t < 2 * 64 and (wanted > 0 or more_w == 0)
    for singles in range(1, 70):
        more_s, more_o, more_t, more_w = runner._fill(singles, 0, 0, singles)
        assert more_o == more_t == 0
        if singles <= 8:
            assert more_s == more_w == 0
        else:
            assert (singles + more_s) % 8 == 0 and (singles + more_w) % 8 == 0


def test_threads_submit_while_the_loop_thread_runs(models):
    """Several caller threads submit requests and wait for them while the engine's own thread
    drives the loop: every request gets the tokens it gets alone, and the engine ends clean."""
    import threading

    folder, loaded, plain = models["B"]
    config, _, page = CONFIGS["B"]
    engine = Engine(loaded, cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=512),
                    batching_config=BatchingConfig(max_sequences=3, queue_size=32,
                                                   prefill_chunk_size=8, max_scheduled_tokens=16,
                                                   loop_thread=True))
    requests = prompts(config["vocab_size"], (3, 17, 9, 30, 1, 12, 25, 6), seed=21)
    results, errors = {}, []

    def caller(numbers):
        try:
            for number in numbers:
                handle = engine.submit_ids(requests[number], max_tokens=5, ignore_eos=True)
                results[number] = list(handle.result().token_ids)
        except BaseException as error:          # noqa: BLE001
            errors.append(error)

    threads = [threading.Thread(target=caller, args=(range(start, 8, 3),)) for start in range(3)]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join(timeout=120)
    assert not errors and not any(thread.is_alive() for thread in threads)
    for number, prompt in enumerate(requests):
        assert results[number] == plain.greedy(prompt, 5)
    engine.close()
    assert not engine.cache.requests() and engine._thread is None
