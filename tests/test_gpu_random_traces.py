"""Seeded random traces through the replay engine (the one `bin/trace_run` drives): three to
seven requests of 2 to 420 tokens, at most four live, fed in portions of 1, 2-9 or 10-150 tokens,
some left out of a step, logits wanted at random places, and a cache that holds just what the
live requests need (each rounded up to 64 tokens), so that pages are used again. Every wanted
row is compared with the plain implementation, in both dtypes."""

import random

import pytest
import torch

from plain_lfm2 import PlainModel
from tiny_models import ALL_CONFIGS, make_model_dir, tolerance

pytestmark = pytest.mark.gpu


def random_trace(rng, vocab):
    longest = rng.choice([60, 200, 420])
    lengths = [rng.choice([rng.randint(2, 30), rng.randint(30, longest)])
               for _ in range(rng.randint(3, 7))]
    requests = {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}
    waiting, live, steps = list(requests), {}, []
    while waiting or live:
        while waiting and len(live) < 4 and rng.random() < 0.7:
            live[waiting.pop(0)] = 0
        if not live:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for request_id in list(live):
            if rng.random() < 0.2 and len(live) > 1:
                continue                                  # left out of this step
            tokens, fed = requests[request_id], live[request_id]
            kind = rng.random()
            size = 1 if kind < 0.35 else rng.randint(2, 9) if kind < 0.7 else rng.randint(10, 150)
            size = min(size, len(tokens) - fed)
            want = sorted(rng.sample(range(size), rng.randint(0, min(size, 3))))
            if fed + size == len(tokens) and size - 1 not in want:
                want.append(size - 1)
            entries.append({"id": request_id, "tokens": tokens[fed:fed + size], "want": want,
                            "at": fed})
            live[request_id] = fed + size
            if live[request_id] == len(tokens):
                end.append(request_id)
                del live[request_id]
        if entries:
            steps.append((entries, end))
    return requests, steps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("trace_models")
    return {name: make_model_dir(name, root) for name in ALL_CONFIGS}


@pytest.mark.parametrize("seed", range(10))
def test_random_trace(folders, seed):
    from mlx_one_b200.engine.replay import Replay

    name = list(ALL_CONFIGS)[seed % len(ALL_CONFIGS)]
    config = ALL_CONFIGS[name][0]
    rng = random.Random(seed)
    requests, steps = random_trace(rng, config["vocab_size"])
    plain = PlainModel(folders[name])
    expected = {request_id: plain.logits(tokens) for request_id, tokens in requests.items()}
    held, most = {}, 0
    for entries, end in steps:
        for entry in entries:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        most = max(most, sum(-(-n // 64) * 64 for n in held.values()))
        for request_id in end:
            del held[request_id]
    compared = 0
    for dtype in ("float32", "bfloat16"):
        replay = Replay(folders[name], dtype=dtype, max_tokens=most, page_size=16)
        kind = torch.float32 if dtype == "float32" else torch.bfloat16
        bounds = {request_id: tolerance(kind, logits) for request_id, logits in expected.items()}
        for number, (entries, end) in enumerate(steps):
            out = replay.run([{"id": e["id"], "tokens": e["tokens"], "want": e["want"]}
                              for e in entries], end)
            row = 0
            for entry in entries:
                for place in entry["want"]:
                    got = torch.from_numpy(out[row])
                    want = expected[entry["id"]][entry["at"] + place]
                    atol, rtol = bounds[entry["id"]]
                    excess = ((got - want).abs() - (atol + rtol * want.abs())).max().item()
                    assert excess <= 0, (f"{name} {dtype} seed {seed} step {number} request "
                                         f"{entry['id']} position {entry['at'] + place}: over the "
                                         f"tolerance by {excess:.3g}")
                    row += 1
                    compared += 1
            assert out is None or row == out.shape[0]
        assert not replay.cache.requests()
    assert compared > 0
