"""Tiny LFM2 configurations for the tests, and helpers that replay requests.

The configurations differ in every size and option: layer order and first layer kind, hidden
size, head count, key-head groups (2 per key head, all on one key head, 3 per key head), head
size (16, 32, 48, 64), feed-forward rule (given width, auto-adjusted), vocabulary (a power of two
and not), rope theta, convolution width (3, 4, 2) and bias, tied and separate head, norm eps,
and a sliding window in one of them.
"""

from __future__ import annotations

import tempfile
from pathlib import Path

import torch

TINY_A = dict(
    model_type="lfm2", num_hidden_layers=4,
    layer_types=["conv", "full_attention", "conv", "full_attention"],
    hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
    block_auto_adjust_ff_dim=False, block_ff_dim=192, vocab_size=512, rope_theta=10000.0,
    conv_L_cache=3, conv_bias=False, tie_embedding=True, norm_eps=1e-5)

TINY_B = dict(
    model_type="lfm2", num_hidden_layers=6,
    layer_types=["full_attention", "conv", "conv", "full_attention", "conv", "full_attention"],
    hidden_size=96, num_attention_heads=3, num_key_value_heads=1,
    block_auto_adjust_ff_dim=True, block_ff_dim=384, block_multiple_of=64,
    block_ffn_dim_multiplier=1.0, vocab_size=1000, rope_theta=1000000.0,
    conv_L_cache=4, conv_bias=True, tie_embedding=False, norm_eps=1e-6)

TINY_C = dict(
    model_type="lfm2", num_hidden_layers=5,
    layer_types=["conv", "sliding_attention", "full_attention", "sliding_attention", "conv"],
    hidden_size=288, num_attention_heads=6, num_key_value_heads=2,
    block_auto_adjust_ff_dim=True, block_ff_dim=500, block_multiple_of=20,
    block_ffn_dim_multiplier=1.3, vocab_size=777, rope_theta=50000.0, sliding_window=19,
    conv_L_cache=2, conv_bias=False, tie_embedding=True, norm_eps=3e-6)

# head size 64 with pages of 8 keys: prefill attention takes the tcgen05 kernel (two query heads
# stacked per key head, a window inside a key tile), everything else stays tiny
TINY_D = dict(
    model_type="lfm2", num_hidden_layers=4,
    layer_types=["full_attention", "conv", "sliding_attention", "full_attention"],
    hidden_size=128, num_attention_heads=2, num_key_value_heads=1,
    block_auto_adjust_ff_dim=False, block_ff_dim=136, vocab_size=301, rope_theta=20000.0,
    sliding_window=40, conv_L_cache=3, conv_bias=True, tie_embedding=False, norm_eps=2e-5)

# a size at which the kernels for large steps (tcgen05 products, wide conv and q/k kernels) run
MID = dict(
    model_type="lfm2", num_hidden_layers=5,
    layer_types=["conv", "full_attention", "conv", "sliding_attention", "full_attention"],
    hidden_size=512, num_attention_heads=8, num_key_value_heads=2,
    block_auto_adjust_ff_dim=True, block_ff_dim=2000, block_multiple_of=8,
    vocab_size=3001, rope_theta=1000000.0, sliding_window=150, conv_L_cache=3, conv_bias=False,
    tie_embedding=True, norm_eps=1e-5)

CONFIGS = {"A": (TINY_A, 0, 4), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16),
           "D": (TINY_D, 5, 8)}   # config, seed, page
ALL_CONFIGS = {**CONFIGS, "MID": (MID, 3, 16)}

# (atol, rtol) on logits: |engine - plain| <= atol + rtol * |plain|. In 32-bit the bound is the
# reference's for its own parity runs (src/mlx_one/inference_baseline.py:30). Its bfloat16 bound
# (5e-2) is meant for checkpoints whose logits are an order of magnitude larger than those of
# these random models (standard deviation 0.16 to 0.5), where it would be wider than the effect
# of a wrong key. So the bfloat16 bound here is relative to the spread of the plain logits:
# measured rounding of the bfloat16 engine is 1.5 to 5 % of that spread, one wrong prompt token
# moves the last logits by 15 to 60 % of it.
TOLERANCE = {torch.float32: (1e-4, 1e-4), torch.bfloat16: (None, 1e-2)}
BF16_ATOL_OF_SPREAD = 0.08


def tolerance(dtype, want: torch.Tensor) -> tuple[float, float]:
    atol, rtol = TOLERANCE[dtype]
    if atol is None:
        atol = BF16_ATOL_OF_SPREAD * float(want.float().std())
    return atol, rtol


def make_model_dir(name: str, root: Path | None = None, dtype=torch.bfloat16) -> Path:
    """Writes the tiny model ``name`` into a fresh temporary folder (never into the repo)."""
    from mlx_one_b200.weights import write_random_model

    config, seed, _ = ALL_CONFIGS[name]
    folder = Path(tempfile.mkdtemp(prefix=f"tiny_{name}_", dir=root))
    return write_random_model(folder, config, seed, dtype)


def prompts(vocab: int, lengths, seed: int = 0):
    generator = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=generator).tolist() for n in lengths]


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype, what: str = "") -> None:
    got, want = got.float().cpu(), want.float().cpu()
    atol, rtol = tolerance(dtype, want)
    excess = (got - want).abs() - (atol + rtol * want.abs())
    worst = excess.max().item()
    if not worst <= 0:
        index = int(excess.argmax())
        row = index // got.shape[-1] if got.dim() > 1 else 0
        raise AssertionError(
            f"{what}: logits differ by {(got - want).abs().max().item():.3e} "
            f"(allowed {atol} + {rtol}*|ref|), first at row {row}; "
            f"rows over tolerance: {torch.nonzero((excess > 0).any(dim=-1)).flatten().tolist()[:8]}")


def replay(runner, cache, steps):
    """Runs ``steps`` = list of (entries, end) with entries = [(id, tokens)], asking for
    logits everywhere. Returns {id: float32 logits [all its tokens, vocab]} on the host."""
    from mlx_one_b200.engine.runner import StepEntry

    collected: dict = {}
    for entries, end in steps:
        batch = []
        for request_id, tokens in entries:
            if request_id not in cache:
                cache.open(request_id)
            batch.append(StepEntry(request_id, tokens, range(len(tokens))))
        logits = runner.step(batch)
        at = 0
        for request_id, tokens in entries:
            collected.setdefault(request_id, []).append(logits[at:at + len(tokens)].float().cpu())
            at += len(tokens)
        for request_id in end:
            cache.close(request_id)
        cache.check()
    runner.ops.check_errors()
    return {key: torch.cat(parts) for key, parts in collected.items()}


def cut(tokens, sizes):
    """Cuts ``tokens`` into portions of the given sizes, cycling; the rest in one piece."""
    out, at, i = [], 0, 0
    while at < len(tokens):
        size = sizes[i % len(sizes)]
        out.append(tokens[at:at + size])
        at += size
        i += 1
    return out


def mixed_schedule(requests, live_limit=4, decode_tail=8):
    """Steps for a dict id -> tokens: up to ``live_limit`` live requests, prompt portions of
    changing size (down to two tokens) beside single decoded tokens of others, requests
    sometimes left out of a step, and every request ended as soon as its tokens are fed."""
    waiting = list(requests)
    live: dict = {}
    steps, turn = [], 0
    while waiting or live:
        while waiting and len(live) < live_limit:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for slot, request_id in enumerate(list(live)):
            tokens, fed = requests[request_id], live[request_id]
            prompt_part = max(len(tokens) - decode_tail, 1)
            if fed < prompt_part:
                size = min((5, 2, 11, 3)[(turn + slot) % 4], prompt_part - fed)
            else:
                size = 1
            if (turn + slot) % 5 == 4 and fed > 0:
                continue                            # left out of this step, goes on later
            entries.append((request_id, tokens[fed:fed + size]))
            live[request_id] = fed + size
            if live[request_id] == len(tokens):
                end.append(request_id)
                del live[request_id]
        if entries:
            steps.append((entries, end))
        turn += 1
    return steps
