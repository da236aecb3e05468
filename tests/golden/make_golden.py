"""Writes tests/golden/reference_pieces.json from the parts of the reference that can be
imported on a machine without MLX.

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py

The reference's model classes need ``mlx.nn`` and cannot be imported here, so there is no
golden forward pass: the plain implementation (tests/plain_lfm2.py) rests on the formulas in
the reference's source. What can be run are its configuration class, its weight contract, its
convolution cache (with ``mlx.core`` replaced by NumPy, as the reference's own tests do),
its NumPy paged-attention oracle (given stand-ins for its page objects that carry NumPy
arrays), its rotary encoding with explicit positions (``apply_rope`` of
models/shared/transformer.py, which needs only cos, sin, power, arange and concatenate of
``mlx.core``; ``mlx.nn`` is stood in by an empty ``Module``) and its sampling rule. Their
outputs for fixed inputs are stored here and compared with this repository's own code by
tests/test_golden.py. After this, of the model's formulas only ``nn.RMSNorm``, which is MLX's
own and not in the reference's source, rests on reading alone.
"""

import json
import random
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

from tiny_models import TINY_A, TINY_B, TINY_C  # noqa: E402

LFM2_1_2B = dict(
    model_type="lfm2", num_hidden_layers=16, hidden_size=2048, num_attention_heads=32,
    num_key_value_heads=8, block_ff_dim=12288, block_multiple_of=256, vocab_size=65536,
    layer_types=["conv", "conv", "full_attention", "conv", "conv", "full_attention", "conv",
                 "conv", "full_attention", "conv", "full_attention", "conv", "full_attention",
                 "conv", "full_attention", "conv"])


def paged_attention_case():
    """The reference's NumPy oracle (engine/paged_attention.py:209-246) on two requests whose
    pages lie shuffled in one pool: 6 query heads over 2 key heads, head size 8, pages of 4.
    Its page objects are stood in by plain namespaces that pass its own layout checks."""
    from types import SimpleNamespace as Namespace

    from mlx_one.engine.paged import KERNEL_VERSION
    from mlx_one.engine.paged_attention import numpy_paged_attention

    rng = np.random.default_rng(7)
    kv_heads, head_dim, page, heads = 2, 8, 4, 6
    lengths = (11, 6)
    positions = ((8, 9, 10), (5, 0, 0))             # three queries of request 0, one of request 1
    widths = (3, 1)
    pool_pages = 9
    pool = rng.standard_normal((2, pool_pages, kv_heads, page, head_dim)).astype(np.float32)
    tables = [[7, 2, 5], [0, 8]]                    # page numbers in the pool, in logical order
    owner = object()
    rows = []
    for length, table in zip(lengths, tables):
        blocks = []
        for index, number in enumerate(table):
            count = min(page, length - index * page)
            layout = Namespace(version=3, layer_id=0, page_tokens=page, key_dtype="float32",
                               value_dtype="float32", kernel_version=KERNEL_VERSION,
                               quantization_group_size=32, num_kv_heads=kv_heads,
                               head_dim=head_dim, quantization_bits=None)
            block = Namespace(layout=layout, token_count=count, immutable=count == page,
                              state=[pool[0, number][None], pool[1, number][None]])
            blocks.append(Namespace(block=block, pool=owner, block_id=number))
        rows.append(Namespace(_blocks=blocks, offset=length, pool=owner, layer_id=0,
                              block_tokens=page, dtype="float32", bits=None))
    queries = rng.standard_normal((2, heads, 3, head_dim)).astype(np.float32)
    scale = head_dim ** -0.5
    result = numpy_paged_attention(queries, rows, positions, widths, scale=scale)
    return {"kv_heads": kv_heads, "head_dim": head_dim, "page": page, "heads": heads,
            "pool": pool.tolist(), "tables": tables, "lengths": list(lengths),
            "positions": [list(p) for p in positions], "widths": list(widths),
            "queries": queries.tolist(), "scale": scale, "output": result.tolist()}


def rope_cases():
    """The reference's rotary encoding with explicit position_ids
    (models/shared/transformer.py:27-29, 50-51, 67-72, 88-90)."""
    from mlx_one.models.shared.transformer import apply_rope

    rng = np.random.default_rng(11)
    cases = []
    for head_dim, theta, positions in ((8, 10000.0, [0, 1, 2, 77]),
                                       (16, 1000000.0, [5, 6, 900, 4095, 100000])):
        value = rng.standard_normal((1, 3, len(positions), head_dim)).astype(np.float32)
        rotated = apply_rope(value, offset=0, theta=theta, position_ids=np.array([positions]))
        cases.append({"head_dim": head_dim, "theta": theta, "positions": positions,
                      "value": value.tolist(), "rotated": np.asarray(rotated).tolist()})
    return cases


def main():
    out = {}
    from mlx_one.models.language.lfm2.config import Lfm2Config
    from mlx_one.models.language.lfm2.weights import weight_contract

    configs = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "1.2B": LFM2_1_2B,
               "defaults": {"model_type": "lfm2"},
               "idxs": {"model_type": "lfm2", "num_hidden_layers": 6, "full_attn_idxs": [1, 4]}}
    out["config"] = {}
    for name, data in configs.items():
        cfg = Lfm2Config.from_dict(data)
        out["config"][name] = {
            "intermediate": cfg.adjusted_intermediate_size, "layer_types": list(cfg.layer_types),
            "full_attn_idxs": list(cfg.full_attn_idxs), "rope_theta": cfg.rope_theta,
            "tensors": {k: list(v) for k, v in weight_contract(cfg).expected.items()}}
    rejected = {
        "odd_head": {"model_type": "lfm2", "hidden_size": 30, "num_attention_heads": 2,
                     "num_key_value_heads": 2},
        "heads": {"model_type": "lfm2", "hidden_size": 64, "num_attention_heads": 3},
        "groups": {"model_type": "lfm2", "num_attention_heads": 16, "num_key_value_heads": 5},
        "layer_count": {"model_type": "lfm2", "num_hidden_layers": 3, "layer_types": ["conv"]},
        "layer_kind": {"model_type": "lfm2", "num_hidden_layers": 1, "layer_types": ["mamba"]},
        "no_attention": {"model_type": "lfm2", "num_hidden_layers": 2,
                         "layer_types": ["conv", "conv"]},
        "window": {"model_type": "lfm2", "num_hidden_layers": 1,
                   "layer_types": ["sliding_attention"]},
        "swiglu": {"model_type": "lfm2", "block_use_swiglu": False},
        "rope": {"model_type": "lfm2", "rope_parameters": {"rope_type": "llama3"}},
        "model_type": {"model_type": "llama"},
        "eps": {"model_type": "lfm2", "norm_eps": 0},
    }
    out["rejected"] = {}
    for name, data in rejected.items():
        try:
            Lfm2Config.from_dict(data)
            out["rejected"][name] = None
        except ValueError as error:
            out["rejected"][name] = str(error)

    # convolution cache: mlx.core stood in by NumPy, as tests/optimization/test_lfm2_state.py does
    fake = types.ModuleType("mlx.core")
    fake.zeros = lambda shape, dtype=None: np.zeros(shape, dtype=dtype or np.float32)
    fake.concatenate = lambda values, axis=0: np.concatenate(values, axis=axis)
    fake.array = np.array
    # what apply_rope with explicit positions uses
    fake.float32 = np.float32
    fake.arange = lambda *args, dtype=None: np.arange(*args, dtype=dtype)
    fake.power = lambda base, exponent: np.power(np.float32(base), exponent).astype(np.float32)
    fake.cos, fake.sin, fake.broadcast_to = np.cos, np.sin, np.broadcast_to
    layers = types.ModuleType("mlx.nn")
    layers.Module = type("Module", (), {})
    package = types.ModuleType("mlx")
    package.core, package.nn = fake, layers
    sys.modules.setdefault("mlx", package)
    sys.modules["mlx.core"] = fake
    sys.modules["mlx.nn"] = layers
    from mlx_one.core.cache import ConvCache

    rng = np.random.default_rng(0)
    values = rng.standard_normal((1, 11, 3)).astype(np.float32)
    cache = ConvCache(4)
    windows = []
    for start, stop in ((0, 1), (1, 3), (3, 4), (4, 9), (9, 11)):
        windows.append(np.asarray(cache.update(values[:, start:stop])).tolist())
    out["conv_cache"] = {"taps": 4, "values": values.tolist(), "cuts": [1, 2, 1, 5, 2],
                         "windows": windows}

    out["paged_attention"] = paged_attention_case()
    out["rope"] = rope_cases()

    from mlx_one.text.sampling import _sample_probabilities
    from mlx_one.text.schemas import TextGenerationOptions

    cases = []
    rng = np.random.default_rng(1)
    for index, (top_k, top_p) in enumerate(((None, 1.0), (5, 1.0), (None, 0.7), (8, 0.5),
                                            (1, 1.0), (None, 0.999))):
        logits = rng.standard_normal(50).astype(np.float32) * 2
        if index == 3:
            logits[7] = logits[3]          # a tie inside the kept set
        p = np.exp(logits - logits.max())
        p = (p / p.sum()).astype(np.float32)
        options = TextGenerationOptions(temperature=1.0, top_k=top_k, top_p=top_p)
        picks = []
        for seed in range(8):
            picks.append(_sample_probabilities(p, options, random.Random(seed)))
        # the kept set: every token that some uniform draw can return
        kept = set()

        class Fixed:
            def __init__(self, value):
                self.value = value

            def random(self):
                return self.value

        for i in range(2000):
            kept.add(_sample_probabilities(p, options, Fixed(i / 2000.0)))
        cases.append({"probabilities": p.tolist(), "top_k": top_k, "top_p": top_p,
                      "python_random_picks": picks, "kept": sorted(kept)})
    out["sampling"] = cases
    (HERE / "reference_pieces.json").write_text(json.dumps(out, indent=1))
    print("wrote", HERE / "reference_pieces.json")


if __name__ == "__main__":
    main()
