"""Configuration, registry and weights (no GPU)."""

import json

import pytest
import torch

from mlx_one_b200.config import (Architecture, ConfigError, Lfm2Config, get_architecture,
                                 read_config, register_architecture, unregister_architecture)
from mlx_one_b200.architectures.lfm2 import describe
from mlx_one_b200.parts.model import cache_entries, expected_tensors
from mlx_one_b200.parts.base import FixedState, PagedKeyValues
from mlx_one_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, check_names,
                                  load_weights, random_tensors, write_random_model,
                                  write_safetensors)
from tiny_models import TINY_A, TINY_B, TINY_C


def test_config_reads_every_key_and_alias():
    cfg = Lfm2Config.from_dict({**TINY_B, "tie_word_embeddings": True, "num_heads": 3,
                                "some_future_key": 7, "eos_token_id": [7, 9]})
    assert cfg.tie_embedding is False            # the model's own key wins over the alias
    assert cfg.extra == {"some_future_key": 7}
    assert cfg.head_dim == 32 and cfg.kv_dim == 32
    assert cfg.adjusted_intermediate_size == 256
    assert cfg.eos_token_ids == (7, 9)
    assert Lfm2Config.from_dict({"model_type": "lfm2", "tie_word_embeddings": False}).tie_embedding is False
    assert Lfm2Config.from_dict({"model_type": "lfm2", "num_heads": 8,
                                 "num_key_value_heads": 4}).num_attention_heads == 8
    theta = Lfm2Config.from_dict({"model_type": "lfm2", "rope_parameters": {"rope_theta": 5e5}})
    assert theta.rope_theta == 5e5
    round_trip = Lfm2Config.from_dict(cfg.to_dict())
    assert round_trip == cfg


@pytest.mark.parametrize("bad", [
    {"vocab_size": 0}, {"hidden_size": -4}, {"conv_L_cache": 0}, {"conv_bias": "no"},
    {"norm_eps": float("nan")}, {"block_dim": 7}, {"use_pos_enc": False},
    {"num_hidden_layers": 4, "full_attn_idxs": [0], "layer_types": ["conv"] * 3 + ["full_attention"]},
    {"sliding_window": 0, "num_hidden_layers": 1, "layer_types": ["sliding_attention"]},
])
def test_config_rejects(bad):
    with pytest.raises(ConfigError):
        Lfm2Config.from_dict({"model_type": "lfm2", **bad})


def test_registry_resolves_by_model_type(tmp_path):
    entry = get_architecture("lfm2")
    assert entry.config_class is Lfm2Config
    with pytest.raises(ConfigError, match="unknown architecture"):
        get_architecture("not-a-model")
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    architecture, cfg = read_config(tmp_path)
    assert architecture.name == "lfm2" and cfg.hidden_size == 64
    (tmp_path / "config.json").write_text(json.dumps({"hidden_size": 8}))
    with pytest.raises(ConfigError, match="model_type"):
        read_config(tmp_path)
    with pytest.raises(ValueError):
        register_architecture(Architecture("lfm2", Lfm2Config, describe))
    register_architecture(Architecture("lfm2-copy", Lfm2Config, describe))
    try:
        assert get_architecture("lfm2-copy").describe is describe
    finally:
        unregister_architecture("lfm2-copy")


def test_description_chooses_parts_layer_by_layer():
    spec = describe(Lfm2Config.from_dict(TINY_C))
    kinds = [layer.mixer.kind for layer in spec.layers]
    assert kinds == ["short_conv", "attention", "attention", "attention", "short_conv"]
    assert [layer.mixer.get("window") for layer in spec.layers] == [None, 19, None, 19, None]
    assert spec.layers[1].mixer["position"]["theta"] == 50000.0
    assert spec.layers[0].mixer_norm["eps"] == 3e-6
    needs = cache_entries(spec)
    assert needs[0] == FixedState((1, 288)) and needs[4] == FixedState((1, 288))
    assert needs[1] == PagedKeyValues(2, 48, 19) and needs[2] == PagedKeyValues(2, 48, None)
    assert len(expected_tensors(spec)) == 2 + 5 * 5 + 2 * 3 + 3 * 6


def test_safetensors_round_trip_and_errors(tmp_path):
    tensors = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int64),
               "c": torch.randn(2, 2), "empty": torch.zeros(0, 4)}
    path = tmp_path / "x.safetensors"
    write_safetensors(path, tensors, {"k": "v"})
    with SafetensorsFile(path) as handle:
        assert handle.metadata == {"k": "v"}
        for name, value in tensors.items():
            assert torch.equal(handle.tensor(name).clone(), value)
    # the same file read by the library that everybody else uses
    from safetensors.torch import load_file
    for name, value in load_file(str(path)).items():
        assert torch.equal(value, tensors[name])
    (tmp_path / "bad.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{not json")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(tmp_path / "bad.safetensors")
    # headers whose byte ranges run backwards, start before the data or share bytes
    import json
    import struct

    def with_header(header, data=b"\0" * 16):
        raw = json.dumps(header).encode()
        target = tmp_path / "crafted.safetensors"
        target.write_bytes(struct.pack("<Q", len(raw)) + raw + data)
        return target

    entry = lambda begin, end, shape: {"dtype": "F32", "shape": shape, "data_offsets": [begin, end]}
    for header, what in (({"t": entry(-8, 0, [2])}, "inconsistent offsets"),
                         ({"t": entry(8, 0, [-2])}, "inconsistent offsets"),
                         ({"t": entry(0, 8, [2]), "u": entry(4, 12, [2])}, "overlaps")):
        with pytest.raises(SafetensorsError, match=what):
            SafetensorsFile(with_header(header))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    spec = describe(Lfm2Config.from_dict(TINY_A))
    tensors = random_tensors(spec, 0)
    del tensors["model.layers.1.self_attn.q_proj.weight"]
    del tensors["model.embedding_norm.weight"]
    tensors["model.layers.0.conv.extra"] = torch.zeros(2)
    tensors["model.layers.2.ffn_norm.weight"] = torch.zeros(65)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as caught:
        load_weights(tmp_path, spec, torch.bfloat16, "cpu")
    error = caught.value
    assert error.missing == ("model.embedding_norm.weight", "model.layers.1.self_attn.q_proj.weight")
    assert error.unexpected == ("model.layers.0.conv.extra",)
    assert error.mismatched == (("model.layers.2.ffn_norm.weight", (65,), (64,)),)
    for word in ("missing tensors", "unexpected tensors", "wrong shapes", "q_proj", "extra", "(65,)"):
        assert word in str(error)


def test_renames_and_dropped_tensors(tmp_path):
    """conv.conv.weight [H, 1, L], conv.conv.bias, rotary tables and a tied lm_head, as a
    checkpoint from the original framework stores them."""
    spec = describe(Lfm2Config.from_dict({**TINY_A, "conv_bias": True}))
    tensors = random_tensors(spec, 3)
    stored = {}
    for name, value in tensors.items():
        if name.endswith("conv.conv"):
            stored[name + ".weight"] = value[:, None, :].contiguous()
        elif name.endswith("conv.conv_bias"):
            stored[name[:-len("conv_bias")] + "conv.bias"] = value
        else:
            stored[name] = value
    stored["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    stored["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    write_safetensors(tmp_path / "model.safetensors", stored)
    loaded = load_weights(tmp_path, spec, torch.bfloat16, "cpu")
    assert set(loaded) == set(tensors)
    for name in tensors:
        assert torch.equal(loaded[name], tensors[name]), name


def test_dtypes_are_kept(tmp_path):
    spec = describe(Lfm2Config.from_dict(TINY_A))
    tensors = random_tensors(spec, 0)
    tensors["model.embedding_norm.weight"] = tensors["model.embedding_norm.weight"].float()
    write_safetensors(tmp_path / "model.safetensors", tensors)
    as_bf16 = load_weights(tmp_path, spec, torch.bfloat16, "cpu")
    assert as_bf16["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert as_bf16["model.embedding_norm.weight"].dtype == torch.float32     # stored in 32-bit
    as_f32 = load_weights(tmp_path, spec, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in as_f32.values())
    assert torch.equal(as_f32["model.embed_tokens.weight"],
                       tensors["model.embed_tokens.weight"].float())


def test_random_weights_are_seeded_and_distributed(tmp_path):
    first = write_random_model(tmp_path / "a", TINY_B, seed=1)
    again = write_random_model(tmp_path / "b", TINY_B, seed=1)
    other = write_random_model(tmp_path / "c", TINY_B, seed=2)
    read = lambda folder: (folder / "model.safetensors").read_bytes()
    assert read(first) == read(again) != read(other)
    assert json.loads((first / "config.json").read_text())["conv_L_cache"] == 4
    spec = describe(Lfm2Config.from_dict(TINY_B))
    tensors = random_tensors(spec, 1, torch.float32)
    table = tensors["model.embed_tokens.weight"]
    assert abs(float(table.std()) - 0.02) < 1e-3 and abs(float(table.mean())) < 1e-3
    norm = tensors["model.layers.0.operator_norm.weight"]
    assert abs(float(norm.mean()) - 1) < 0.05 and 0.05 < float(norm.std()) < 0.15
    assert "lm_head.weight" in tensors and "model.layers.1.conv.conv_bias" in tensors
    check_names(spec, {k: tuple(v.shape) for k, v in tensors.items()})


def test_shards_follow_the_index_and_stay_inside_the_folder(tmp_path):
    """The reference's rules for checkpoint files (src/mlx_one/text/loading.py:538-610): shards
    need an index that says where every tensor is; files outside the folder, pickle checkpoints
    and several files without an index are refused."""
    spec = describe(Lfm2Config.from_dict(TINY_A))
    tensors = random_tensors(spec, 4)
    names = sorted(tensors)
    halves = {"model-00001-of-00002.safetensors": names[::2],
              "model-00002-of-00002.safetensors": names[1::2]}
    folder = tmp_path / "sharded"
    folder.mkdir()
    for file, part in halves.items():
        write_safetensors(folder / file, {name: tensors[name] for name in part})
    with pytest.raises(SafetensorsError, match="no index"):
        load_weights(folder, spec, torch.bfloat16, "cpu")
    weight_map = {name: file for file, part in halves.items() for name in part}
    index = folder / "model.safetensors.index.json"
    index.write_text(json.dumps({"weight_map": weight_map}))
    loaded = load_weights(folder, spec, torch.bfloat16, "cpu")
    assert all(torch.equal(loaded[name], tensors[name]) for name in names)
    # a tensor that lies in another shard than the index says; a name that no shard holds
    swapped = dict(weight_map)
    swapped[names[0]] = "model-00002-of-00002.safetensors"
    index.write_text(json.dumps({"weight_map": swapped}))
    with pytest.raises(SafetensorsError, match="not where the index says"):
        load_weights(folder, spec, torch.bfloat16, "cpu")
    index.write_text(json.dumps({"weight_map": {**weight_map, "ghost.weight": next(iter(halves))}}))
    with pytest.raises(SafetensorsError, match="in no shard"):
        load_weights(folder, spec, torch.bfloat16, "cpu")
    index.write_text(json.dumps({"weight_map": {}}))
    with pytest.raises(SafetensorsError, match="weight_map"):
        load_weights(folder, spec, torch.bfloat16, "cpu")
    index.write_text(json.dumps({"weight_map": {**weight_map, names[0]: "gone.safetensors"}}))
    with pytest.raises(FileNotFoundError, match="named by the index"):
        load_weights(folder, spec, torch.bfloat16, "cpu")
    index.write_text(json.dumps({"weight_map": {**weight_map, names[0]: "../model.safetensors"}}))
    with pytest.raises(FileNotFoundError, match="named by the index"):
        load_weights(folder, spec, torch.bfloat16, "cpu")
    # a shard that is a link to a file elsewhere
    outside = tmp_path / "elsewhere.safetensors"
    write_safetensors(outside, tensors)
    linked = tmp_path / "linked"
    linked.mkdir()
    (linked / "model.safetensors").symlink_to(outside)
    with pytest.raises(SafetensorsError, match="inside"):
        load_weights(linked, spec, torch.bfloat16, "cpu")
    # pickle checkpoints are named in the error, not read
    pickled = tmp_path / "pickled"
    pickled.mkdir()
    (pickled / "pytorch_model.bin").write_bytes(b"\x80\x02")
    with pytest.raises(FileNotFoundError, match="pickle checkpoints"):
        load_weights(pickled, spec, torch.bfloat16, "cpu")
