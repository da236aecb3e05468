"""Text prompts (tokenizer, BOS rule, stop strings, streaming hold-back) on the CPU with the
plain kernel restatements, and the command line on the GPU."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions
from mlx_one_b200.engine.loading import load_model
from plain_lfm2 import PlainModel
from plain_ops import PlainOps
from tiny_models import TINY_A, make_model_dir

ROOT = Path(__file__).resolve().parent.parent
WORDS = ["<bos>", "<eos>"] + [f"w{i}" for i in range(510)]


def folder_with_tokenizer(tmp_path, dtype=torch.float32):
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit

    from mlx_one_b200.weights import write_random_model

    config = {**TINY_A, "bos_token_id": 0, "eos_token_id": 1}
    folder = write_random_model(tmp_path / "model", config, seed=0, dtype=dtype)
    tokenizer = Tokenizer(WordLevel({word: i for i, word in enumerate(WORDS)}, unk_token="w0"))
    tokenizer.pre_tokenizer = WhitespaceSplit()
    tokenizer.save(str(folder / "tokenizer.json"))
    return folder


def test_text_generation_with_bos_stop_and_streaming(tmp_path):
    folder = folder_with_tokenizer(tmp_path)
    loaded = load_model(folder, "float32", "cpu", ops=PlainOps())
    engine = Engine(loaded, cache_config=CacheConfig(block_size_tokens=4, capacity_tokens=256),
                    batching_config=BatchingConfig(max_sequences=2))
    assert engine.encode("w5 w17 w3") == [0, 7, 19, 5]                 # BOS put in front
    assert engine.encode("<bos> w5") == [0, 7]                         # but never twice
    plain = PlainModel(folder)
    expected = plain.greedy([0, 7, 19, 5], 6)
    result = engine.generate("w5 w17 w3", max_tokens=6)
    assert list(result.token_ids) == expected and result.prompt_tokens == 4
    assert result.text == " ".join(WORDS[t] for t in expected)
    assert json.loads(result.to_json())["finish_reason"] == "length"
    assert not engine.cache.requests()
    with pytest.raises(ValueError):
        engine.generate("w5", TextGenerationOptions(max_tokens=2), temperature=0.5)
    with pytest.raises(ValueError):
        TextGenerationOptions(top_p=0.0)


def text_engine(tmp_path, **batching):
    folder = folder_with_tokenizer(tmp_path)
    loaded = load_model(folder, "float32", "cpu", ops=PlainOps())
    engine = Engine(loaded, cache_config=CacheConfig(block_size_tokens=4, capacity_tokens=256),
                    batching_config=BatchingConfig(max_sequences=2, **batching))
    return engine, PlainModel(folder)


@pytest.mark.parametrize("how", ["generate", "submit", "async", "stream", "loop_thread"])
def test_a_stop_string_ends_the_request_where_it_is_committed(tmp_path, how):
    """On every way in, a stop string ends the request at the token that completes it: the
    reason is "stop", only the tokens before the match are counted and no further step runs
    (src/mlx_one/text/generation.py:266-290, 682-697 of the reference)."""
    import asyncio

    engine, plain = text_engine(tmp_path, loop_thread=how == "loop_thread")
    prompt, prompt_ids = "w5 w17 w3", [0, 7, 19, 5]
    # greedy decoding of this tiny model repeats one word; a seeded draw gives different ones
    for seed in range(50):
        sampling = dict(temperature=1.0, seed=seed)
        expected = engine.generate(prompt, max_tokens=6, **sampling).token_ids
        words = [WORDS[t] for t in expected]
        if len(set(words)) == 6 and not {"<bos>", "<eos>"} & set(words):
            break
    else:
        raise AssertionError("no seed gave six different words")

    def ask(stop):
        options = TextGenerationOptions(max_tokens=6, stop=stop, **sampling)
        before = engine.runtime_stats()["tokens_run"]
        if how in ("generate", "loop_thread"):
            result = engine.generate(prompt, options)
        elif how == "submit":
            result = engine.submit(prompt, options).result()
        elif how == "async":
            result = asyncio.run(engine.async_generate(prompt, options=options))
        else:
            chunks = list(engine.stream(prompt, options))
            assert all(c.finish_reason is None for c in chunks[:-1])
            return ("".join(c.text for c in chunks), chunks[-1].finish_reason,
                    chunks[-1].generated_tokens, engine.runtime_stats()["tokens_run"] - before)
        return (result.text, result.finish_reason, result.generation_tokens,
                engine.runtime_stats()["tokens_run"] - before)

    # the first token completes the stop string: nothing is kept, one step ran (the prompt)
    assert ask((words[0],)) == ("", "stop", 0, len(prompt_ids))
    # a token in the middle: the tokens before it are kept; prompt + 2 decode steps ran
    text, reason, count, ran = ask((words[2],))
    assert (text.strip(), reason, count) == (" ".join(words[:2]), "stop", 2)
    assert ran == len(prompt_ids) + 2
    # a stop string over two tokens: both are taken back
    text, reason, count, ran = ask((f"{words[1]} {words[2]}",))
    assert (text.strip(), reason, count) == (words[0], "stop", 1) and ran == len(prompt_ids) + 2
    # no match: all tokens, reason "length"
    assert ask(("never",)) == (" ".join(words), "length", 6, len(prompt_ids) + 5)
    assert not engine.cache.requests()
    engine.close()


def test_stop_strings_need_a_tokenizer(tmp_path):
    loaded = load_model(make_model_dir("A", tmp_path, dtype=torch.float32), "float32", "cpu",
                        ops=PlainOps())
    engine = Engine(loaded, cache_config=CacheConfig(block_size_tokens=4, capacity_tokens=64))
    with pytest.raises(ValueError, match="tokenizer"):
        engine.generate_ids([1, 2], TextGenerationOptions(max_tokens=2, stop=("x",)))


def test_a_kernel_fault_fails_the_requests_of_its_step(tmp_path):
    """The device's error flag travels to the host with the chosen tokens. A step that finds
    it set commits nothing: its requests raise the fault, their pages come back, and the
    engine goes on with other requests. ``close`` reports a fault nobody has read."""
    engine, plain = text_engine(tmp_path)
    ops = engine.model.ops
    prompt_ids = [0, 7, 19, 5]
    handle = engine.submit_ids(prompt_ids, TextGenerationOptions(max_tokens=6))
    other = engine.submit_ids(prompt_ids, TextGenerationOptions(max_tokens=4))
    for _ in range(3):
        engine.step()
    ops.error_flag.fill_(9)
    with pytest.raises(RuntimeError, match="kernel reported"):
        handle.result()
    with pytest.raises(RuntimeError, match="kernel reported"):
        other.result()
    assert int(ops.error_flag.item()) == 0 and not engine.cache.requests()
    assert engine.runtime_stats()["kernel_faults"] == 1
    again = engine.generate_ids(prompt_ids, TextGenerationOptions(max_tokens=6))
    assert list(again.token_ids) == plain.greedy(prompt_ids, 6)
    ops.error_flag.fill_(3)
    with pytest.raises(RuntimeError, match="kernel reported"):
        engine.close()
    assert not engine.cache.requests()


def test_the_loop_thread_serves_handles_that_nobody_drives(tmp_path):
    """With ``loop_thread`` a submitted request finishes although its caller only polls
    ``done()``; ``tokens()`` hands out the tokens as they are committed."""
    import time

    engine, plain = text_engine(tmp_path, loop_thread=True)
    prompt_ids = [0, 7, 19, 5]
    first = engine.submit_ids(prompt_ids, TextGenerationOptions(max_tokens=6))
    second = engine.submit_ids(prompt_ids[:3], TextGenerationOptions(max_tokens=5))
    deadline = time.monotonic() + 60
    while not (first.done() and second.done()):
        assert time.monotonic() < deadline
        time.sleep(0.002)
    assert list(first.result().token_ids) == plain.greedy(prompt_ids, 6)
    assert list(second.result().token_ids) == plain.greedy(prompt_ids[:3], 5)
    third = engine.submit_ids(prompt_ids, TextGenerationOptions(max_tokens=6))
    assert list(third.tokens()) == plain.greedy(prompt_ids, 6)
    engine.close()
    assert not engine.cache.requests()
    # without the thread the caller's iteration drives the loop
    engine, plain = text_engine(tmp_path / "second")
    handle = engine.submit_ids(prompt_ids, TextGenerationOptions(max_tokens=6))
    assert not handle.done()
    assert list(handle.tokens()) == plain.greedy(prompt_ids, 6)


def test_engine_without_tokenizer_asks_for_token_ids(tmp_path):
    loaded = load_model(make_model_dir("A", tmp_path, dtype=torch.float32), "float32", "cpu",
                        ops=PlainOps())
    engine = Engine(loaded, cache_config=CacheConfig(block_size_tokens=4, capacity_tokens=64))
    with pytest.raises(ValueError, match="token ids"):
        engine.generate("hello")
    with pytest.raises(ValueError):
        engine.generate_ids([])
    assert engine.capabilities()["architecture"] == "lfm2"


def test_the_reference_names_for_fetching_a_model(tmp_path):
    """``revision``, ``offline`` and ``cache_dir`` are accepted for a local folder; a name that
    is no folder and a revision are refused; ``tokenizer_source`` names a tokenizer elsewhere."""
    folder = folder_with_tokenizer(tmp_path)
    elsewhere = tmp_path / "tokenizer_only"
    elsewhere.mkdir()
    (folder / "tokenizer.json").rename(elsewhere / "tokenizer.json")
    with pytest.raises(FileNotFoundError, match="no model folder"):
        Engine("LiquidAI/LFM2-1.2B", offline=True, device="cpu", ops=PlainOps())
    with pytest.raises(ValueError, match="revision"):
        Engine(folder, revision="main", device="cpu", ops=PlainOps())
    with pytest.raises(FileNotFoundError, match="tokenizer_source"):
        Engine(folder, tokenizer_source=tmp_path / "nowhere", execution_dtype="float32",
               device="cpu", ops=PlainOps())
    for source in (elsewhere, elsewhere / "tokenizer.json"):
        engine = Engine(folder, offline=True, cache_dir=tmp_path / "unused", tokenizer_source=source,
                        execution_dtype="float32", device="cpu", ops=PlainOps(),
                        cache_config=CacheConfig(block_size_tokens=4, capacity_tokens=64))
        assert engine.encode("w5 w17") == [0, 7, 19]


@pytest.mark.gpu
def test_command_line_generates(tmp_path):
    folder = folder_with_tokenizer(tmp_path, dtype=torch.bfloat16)
    plain = PlainModel(folder)
    run = lambda *args: subprocess.run([sys.executable, str(ROOT / "bin" / "mlx-one"), *args],
                                       capture_output=True, text=True, timeout=600)
    by_ids = run("generate", str(folder), "0 7 19 5", "--token-ids", "--max-tokens", "5",
                 "--dtype", "float32", "--offline", "--cache-dir", str(tmp_path / "unused"))
    assert by_ids.returncode == 0, by_ids.stderr
    assert [int(t) for t in by_ids.stdout.split()] == plain.greedy([0, 7, 19, 5], 5)
    as_json = run("generate", str(folder), "w5 w17 w3", "--max-tokens", "4", "--json-output",
                  "--temperature", "0.7", "--top-k", "20", "--top-p", "0.9", "--seed", "4")
    assert as_json.returncode == 0, as_json.stderr
    payload = json.loads(as_json.stdout)
    assert payload["generation_tokens"] == 4 and payload["prompt_tokens"] == 4
    streamed = run("generate", str(folder), "w5 w17 w3", "--max-tokens", "3", "--stream",
                   "--dtype", "float32")
    assert streamed.returncode == 0 and len(streamed.stdout.split()) == 3
    # a stop string ends the request where it matches, also without --stream
    free = json.loads(run("generate", str(folder), "w5 w17 w3", "--max-tokens", "6",
                          "--json-output", "--temperature", "1.0", "--seed", "3",
                          "--dtype", "float32").stdout)
    words = free["text"].split()
    if len(words) > 2 and words[2] not in words[:2]:
        stopped = run("generate", str(folder), "w5 w17 w3", "--max-tokens", "6", "--json-output",
                      "--temperature", "1.0", "--seed", "3", "--dtype", "float32",
                      "--stop", words[2])
        payload = json.loads(stopped.stdout)
        assert payload["finish_reason"] == "stop" and payload["generation_tokens"] == 2
        assert payload["text"].split() == words[:2]
    bad = run("generate", str(tmp_path / "missing"), "x")
    assert bad.returncode != 0 and "Error" in bad.stderr
