"""Small twins of bench.py's two further workloads, run by the same functions on tiny models and
checked token by token against the plain implementation: continuous batching of 40 requests
through the scheduler, and one long prompt in large portions followed by decoding."""

import sys
from pathlib import Path

import pytest
import torch

from plain_lfm2 import PlainModel
from tiny_models import CONFIGS, make_model_dir

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

pytestmark = pytest.mark.gpu


def greedy_with_margins(plain, prompt, count):
    """The plain model's greedy tokens and, for each, by how much its logit leads."""
    ids, tokens, margins = list(prompt), [], []
    for _ in range(count):
        top = torch.topk(plain.logits(ids)[-1], 2)
        tokens.append(int(top.indices[0]))
        margins.append(float(top.values[0] - top.values[1]))
        ids.append(tokens[-1])
    return tokens, margins


def check_tokens(plain, prompt, got, dtype, what):
    """32-bit: every token equals the plain model's. bfloat16: a token may differ only where
    the plain model's two best logits lie closer than rounding moves them; the request is
    compared no further then."""
    want, margins = greedy_with_margins(plain, prompt, len(got))
    for place, (a, b, margin) in enumerate(zip(got, want, margins)):
        if a != b:
            assert dtype == "bfloat16" and margin < 0.02, (
                f"{what}: token {place} is {a}, the plain model says {b} (margin {margin:.3g})")
            return place
    return len(got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_continuous_batching_of_forty_requests(tmp_path, dtype):
    import bench
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine

    config, _, page = CONFIGS["A"]
    folder = make_model_dir("A", tmp_path)
    plain = PlainModel(folder)
    sequences = 12
    engine = Engine(folder, execution_dtype=dtype, device="cuda:0",
                    cache_config=CacheConfig(block_size_tokens=page,
                                             capacity_tokens=sequences * 128),
                    batching_config=BatchingConfig(max_sequences=sequences, queue_size=40,
                                                   prefill_chunk_size=32, max_prefill_tokens=32,
                                                   max_scheduled_tokens=32 + sequences, timeout=0))
    workload = bench.batching_workload(config["vocab_size"], 40, (2, 160), (2, 24), seed=3)
    results, seconds, records = bench.run_batching(engine, workload)
    engine.model.ops.check_errors()
    phases, histogram = bench.summarize_steps(records)
    assert {"prefill", "mixed", "decode"} <= set(phases)            # all three kinds of step ran
    assert max(r["prompt_tokens"] for r in records) <= 32
    assert max(r["batch_size"] for r in records) <= sequences
    assert sum(histogram.values()) == len(records)
    stats = engine.runtime_stats()
    # forty requests went through a pool that holds twelve: pages were used again
    assert sum(len(p) + n for p, n in workload) > sequences * 128
    assert stats["pages_free"] == stats["pages_total"] and stats["running"] == 0
    compared = 0
    for number, ((prompt, new), result) in enumerate(zip(workload, results)):
        assert result.generation_tokens == new and result.prompt_tokens == len(prompt)
        compared += check_tokens(plain, prompt, list(result.token_ids), dtype, f"request {number}")
    assert compared >= 0.8 * sum(n for _, n in workload)
    engine.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_large_portions_then_decoding(tmp_path, dtype):
    """3000 tokens of the head-size-64 model in portions of 512 through the scheduler (hundreds
    of pages in the block table, steps too large to be captured as graphs), then 12 decoded
    tokens, beside a second request that arrives with it."""
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions
    from tiny_models import prompts

    config, _, page = CONFIGS["D"]
    folder = make_model_dir("D", tmp_path)
    plain = PlainModel(folder)
    engine = Engine(folder, execution_dtype=dtype, device="cuda:0",
                    cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=2 * 3072),
                    batching_config=BatchingConfig(max_sequences=2, queue_size=2,
                                                   prefill_chunk_size=512, max_prefill_tokens=512,
                                                   max_scheduled_tokens=514, timeout=0))
    long_prompt, short_prompt = prompts(config["vocab_size"], (3000, 700), seed=41)
    options = TextGenerationOptions(max_tokens=12)
    results = engine.generate_batch_ids([long_prompt, short_prompt], options)
    engine.model.ops.check_errors()
    traces = engine.step_traces()
    assert max(t["prompt_tokens"] for t in traces) == 512
    assert sum(t["prompt_tokens"] for t in traces) == 3700
    for prompt, result, what in zip((long_prompt, short_prompt), results, ("long", "short")):
        assert check_tokens(plain, prompt, list(result.token_ids), dtype, what) >= 6
    engine.close()
