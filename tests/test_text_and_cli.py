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
    # a stop string cuts the text and ends the request
    stop = WORDS[expected[2]]
    stopped = engine.generate("w5 w17 w3", TextGenerationOptions(max_tokens=6, stop=(stop,)))
    assert stop not in stopped.text and stopped.text == result.text[:result.text.find(stop)]
    chunks = list(engine.stream("w5 w17 w3", max_tokens=6, stop=(stop,)))
    assert chunks[-1].finish_reason == "stop"
    assert "".join(c.text for c in chunks) == stopped.text
    assert not engine.cache.requests()
    with pytest.raises(ValueError):
        engine.generate("w5", TextGenerationOptions(max_tokens=2), temperature=0.5)
    with pytest.raises(ValueError):
        TextGenerationOptions(top_p=0.0)


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
    bad = run("generate", str(tmp_path / "missing"), "x")
    assert bad.returncode != 0 and "Error" in bad.stderr
