"""Decode steps with programmatic dependent launches (a kernel may start, and fetch its
weights, while its predecessor finishes) give the same logits as without."""

import pytest
import torch

from tiny_models import CONFIGS, make_model_dir, prompts

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "C"])
def test_same_logits_with_dependent_launches(tmp_path, name):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner, StepEntry

    config, _, page = CONFIGS[name]
    loaded = load_model(make_model_dir(name, tmp_path), torch.bfloat16, "cuda:0")
    ops = loaded.model.ops
    requests = prompts(config["vocab_size"], (40, 15, 77), seed=9)
    results = []
    try:
        for enabled in (False, True):
            ops.set_dependent_launches(enabled)
            cache = CacheManager(loaded.model.cache_needs, page_size=page, capacity_tokens=512,
                                 max_requests=4, dtype=torch.bfloat16, device="cuda:0")
            runner = Runner(loaded.model, cache)
            for i in range(len(requests)):
                cache.open(i)
            runner.step([StepEntry(i, tokens[:-12]) for i, tokens in enumerate(requests)])
            collected = []
            for step in range(12):       # eager first, then captured as a graph and replayed
                entries = [StepEntry(i, [tokens[len(tokens) - 12 + step]], (0,))
                           for i, tokens in enumerate(requests)]
                collected.append(runner.step(entries).float().cpu().clone())
            ops.check_errors()
            assert runner.graph_replays >= 10
            results.append(torch.stack(collected))
    finally:
        ops.set_dependent_launches(True)
    assert torch.equal(results[0], results[1])
