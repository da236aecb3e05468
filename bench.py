#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on the LFM2-1.2B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096]
                    [--layers L] [--impl ours|reference]

Prints ONE JSON line. ``value`` is decoded tokens per second at the given batch, timed on the
device over exactly K decode steps (each a CUDA-graph replay of the engine's own step, the
chosen token fed to the next step on the device). ``e2e`` is the same through the Python
entry point (``Engine.step``), token ids crossing the host in both directions every step.
``prefill`` is one 2,048-token prompt through the step function. ``roofline`` relates the
decode step to the bytes it has to read: every weight once and the cache of the live
requests. ``points`` holds decode at batch 1 and 64.

Data: seeded uniform-random token ids and N(0, 0.02) weights (norms 1 + N(0, 0.1)); there
are no checkpoints offline. Working set per step (2.3 GB of weights) is far larger than L2,
so no flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# BASELINE.json configs[2]: LFM2-1.2B
LFM2_1_2B = dict(
    model_type="lfm2", num_hidden_layers=16,
    layer_types=["conv", "conv", "full_attention", "conv", "conv", "full_attention", "conv",
                 "conv", "full_attention", "conv", "full_attention", "conv", "full_attention",
                 "conv", "full_attention", "conv"],
    hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
    block_auto_adjust_ff_dim=True, block_ff_dim=12288, block_multiple_of=256,
    block_ffn_dim_multiplier=1.0, vocab_size=65536, rope_theta=1000000.0, conv_L_cache=3,
    conv_bias=False, tie_embedding=True, norm_eps=1e-5, max_position_embeddings=128000)
PAGE_SIZE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in data.items() if k in out})
            out["source"] = "measured"
            return out
        except (ValueError, TypeError):
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._process = None
        self._thread = None

    def start(self):
        try:
            self._process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _read(self):
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self._process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                self.samples.append(float(parts[0]))
                self.max_mhz = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    self.reasons.add(name)

    def stop(self):
        if self._process is not None:
            self._process.terminate()
            try:
                self._process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._process.kill()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def reference_arm():
    """The reference is Apple-MLX only: it pins mlx / mlx-metal wheels that exist for macOS
    on Apple silicon, and its model classes import mlx.nn. Nothing of it can run here."""
    reason = ("reference needs Apple MLX (mlx==0.32.2, mlx-metal; Metal GPU); no wheel exists "
              "for Linux/CUDA and none is in the offline wheelhouse")
    marker = ROOT / "baseline" / "_ref"
    if marker.is_dir():
        try:
            sys.path.insert(0, str(marker))
            import mlx.core  # noqa: F401
            reason = "mlx imported but the reference has no CUDA path; not run"
        except Exception as error:           # noqa: BLE001
            reason += f" (import mlx: {type(error).__name__})"
    print(json.dumps({"impl": "reference", "unavailable": reason}))
    return 0


def build_engine(config, layers, batch, context, steps_ahead):
    import torch

    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine
    from mlx_one_b200.config import get_architecture
    from mlx_one_b200.engine.loading import LoadedModel, build_model
    from mlx_one_b200.weights import random_tensors

    data = dict(config)
    if layers < data["num_hidden_layers"]:
        data["layer_types"] = data["layer_types"][:layers]
        data["num_hidden_layers"] = layers
    architecture = get_architecture(data["model_type"])
    typed = architecture.config_class.from_dict(data)
    spec = architecture.describe(typed)
    tensors = random_tensors(spec, seed=0, dtype=torch.bfloat16, device="cuda:0")
    model = build_model(spec, tensors, "bfloat16", "cuda:0")
    del tensors
    loaded = LoadedModel(Path("random-lfm2-1.2b"), architecture, typed, spec, model)
    capacity = batch * (-(-(context + steps_ahead + 128) // 64) * 64) + PREFILL_TOKENS + 64
    engine = Engine(loaded,
                    cache_config=CacheConfig(block_size_tokens=PAGE_SIZE, capacity_tokens=capacity,
                                             max_requests=batch + 1),
                    batching_config=BatchingConfig(max_sequences=batch, queue_size=batch + 1,
                                                   prefill_chunk_size=2048,
                                                   max_scheduled_tokens=4096,
                                                   max_prefill_tokens=4096))
    return engine


def model_flops(spec, tokens):
    """Matrix-product and attention flops of one whole-prompt step (one logits row)."""
    from mlx_one_b200.parts.model import expected_tensors

    flops = 0
    for name, tensor in expected_tensors(spec).items():
        if len(tensor.shape) == 2 and name != spec.embedding and name != spec.head \
                and not name.endswith("conv.conv"):
            flops += 2 * tokens * tensor.shape[0] * tensor.shape[1]
    flops += 2 * spec.vocab_size * spec.hidden_size          # one row of logits
    for layer in spec.layers:
        if layer.mixer.kind == "attention":
            width = layer.mixer["heads"] * layer.mixer["head_dim"]
            flops += 4 * width * tokens * (tokens + 1) // 2   # causal QK^T and PV
    return flops


def random_prompts(vocab, count, length, seed):
    import torch

    generator = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=generator).tolist() for _ in range(count)]


def fill_requests(engine, prompts, ids):
    """Runs the prompts through the step function, several requests a step, and returns the
    first decoded token of each."""
    from mlx_one_b200.engine.runner import StepEntry

    runner, cache = engine._runner, engine.cache
    firsts = {}
    chunk = 1024
    for request_id in ids:
        cache.open(request_id)
    longest = max(len(p) for p in prompts)
    group = max(1, 4096 // chunk)
    for base in range(0, len(ids), group):
        members = list(range(base, min(base + group, len(ids))))
        for at in range(0, longest, chunk):
            entries = []
            for m in members:
                part = prompts[m][at:at + chunk]
                if part:
                    last = at + chunk >= len(prompts[m])
                    entries.append(StepEntry(ids[m], part, (len(part) - 1,) if last else ()))
            logits = runner.step(entries)
            if logits is not None:
                chosen = engine.model.ops.argmax(logits).tolist()
                for entry, token in zip([e for e in entries if e.want], chosen):
                    firsts[entry.request_id] = token
    return [firsts[i] for i in ids]


def time_decode(engine, batch, context, warmup, steps, seed, sampler=None):
    """Device-timed decode: ``steps`` graph replays after ``warmup``; contexts end at
    ``context``. Returns (seconds, launches per step, mean context)."""
    import torch

    from mlx_one_b200.engine.runner import StepEntry

    vocab = engine.model.spec.vocab_size
    prompt_length = context - warmup - steps - 1
    ids = [f"decode{batch}_{i}" for i in range(batch)]
    prompts = random_prompts(vocab, batch, prompt_length, seed)
    firsts = fill_requests(engine, prompts, ids)
    runner = engine._runner
    entries = [StepEntry(i, [t]) for i, t in zip(ids, firsts)]
    before = engine.model.ops.launches
    chosen = runner.decode_steps(entries, max(warmup, 3))
    torch.cuda.synchronize()
    last = chosen[-1].tolist()
    # launches of one eager step = what the first call launched before it captured
    entries = [StepEntry(i, [t]) for i, t in zip(ids, last)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.start()
        time.sleep(0.25)
    torch.cuda.synchronize()
    start.record()
    runner.decode_steps(entries, steps)
    stop.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(stop) / 1e3
    clocks = sampler.stop() if sampler else None
    mean_context = context - 1 - steps / 2
    for request_id in ids:
        engine.cache.close(request_id)
    return seconds, clocks, mean_context, engine.model.ops.launches - before


def count_step_launches(engine, batch):
    """Kernels that one decode step launches (counted on an eager step of a fresh shape)."""
    import torch

    from mlx_one_b200.engine.runner import StepEntry

    runner, cache, ops = engine._runner, engine.cache, engine.model.ops
    ids = [f"count{i}" for i in range(batch)]
    for request_id in ids:
        cache.open(request_id)
    runner.step([StepEntry(i, [1, 2, 3]) for i in ids])
    graphs, runner.use_graphs = runner.use_graphs, False
    before = ops.launches
    logits = runner.step([StepEntry(i, [4], (0,)) for i in ids])
    ops.argmax(logits)
    launched = ops.launches - before
    runner.use_graphs = graphs
    torch.cuda.synchronize()
    for request_id in ids:
        cache.close(request_id)
    return launched


def time_e2e(engine, batch, context, warmup, steps, seed):
    """Through Engine.step: host token ids in (pinned metadata copy) and out every step."""
    import torch

    from mlx_one_b200 import TextGenerationOptions

    vocab = engine.model.spec.vocab_size
    # prompts finish one after the other (long ones in several portions), so the first request
    # has decoded some tokens when the last one starts; `slack` keeps every request decoding
    # through the timed steps
    slack = batch * (context // PREFILL_TOKENS + 2) + 8
    prompt_length = context - warmup - steps - slack
    prompts = random_prompts(vocab, batch, prompt_length, seed + 1)
    options = TextGenerationOptions(max_tokens=warmup + steps + slack, ignore_eos=True)
    handles = [engine.submit_ids(p, options) for p in prompts]
    from mlx_one_b200.engine.scheduler import Phase
    while any(h.request.phase is not Phase.DECODE for h in handles):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    produced = sum(len(h.request.output) for h in handles)
    began = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - began
    produced = sum(len(h.request.output) for h in handles) - produced
    meta_bytes = engine._runner.last_meta_bytes
    assert produced == batch * steps, (produced, batch, steps)
    for handle in handles:
        handle.cancel()
    engine.step()
    return seconds, meta_bytes


def time_prefill(engine, tokens, warmup, repeats, seed):
    import torch

    from mlx_one_b200.engine.runner import StepEntry

    runner, cache = engine._runner, engine.cache
    prompts = random_prompts(engine.model.spec.vocab_size, warmup + repeats, tokens, seed)
    times = []
    for index, prompt in enumerate(prompts):
        request_id = f"prefill{index}"
        cache.open(request_id)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry(request_id, prompt, (tokens - 1,))])
        stop.record()
        torch.cuda.synchronize()
        if index >= warmup:
            times.append(start.elapsed_time(stop) / 1e3)
        cache.close(request_id)
    return statistics.median(times)


def kernel_case(name: str, batch: int, context: int) -> int:
    """Runs one kernel of the step alone a few times at the benchmark's sizes and prints its
    time: the case that the ncu summaries under profiles/ were captured on."""
    import math

    import torch

    from mlx_one_b200.kernels import default_ops
    from mlx_one_b200.parts.base import PagedKeyValues, PagedView, StepContext

    ops, device = default_ops("cuda:0"), "cuda:0"
    ops.set_dependent_launches(True)
    hidden, width, heads, kv_heads, head_dim = 2048, 8192, 32, 8, 64
    torch.manual_seed(0)

    def weights(n, k, copies):          # several copies, so that no call finds its weights in L2
        return [(torch.randn(n, k, device=device) / math.sqrt(k)).bfloat16() for _ in range(copies)]

    def batch_context(portions, histories):
        as_int = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        positions, owner, starts = [], [], [0]
        for r, (h, n) in enumerate(zip(histories, portions)):
            positions += list(range(h, h + n))
            owner += [r] * n
            starts.append(starts[-1] + n)
        blocks = [-(-(h + n) // PAGE_SIZE) for h, n in zip(histories, portions)]
        table = torch.full((len(portions), max(blocks)), -1, dtype=torch.int32)
        at = 0
        for r, count in enumerate(blocks):
            table[r, :count] = torch.arange(at, at + count)
            at += count
        ctx = StepContext(tokens=len(positions), requests=len(portions),
                          token_ids=as_int([0] * len(positions)), positions=as_int(positions),
                          token_request=as_int(owner), request_start=as_int(starts),
                          history=as_int(histories), max_portion=max(portions),
                          max_context=max(h + n for h, n in zip(histories, portions)))
        kv = torch.randn(2, at, kv_heads, PAGE_SIZE, head_dim, device=device).bfloat16()
        return ctx, PagedView(kv, table.to(device), PAGE_SIZE, PagedKeyValues(kv_heads, head_dim))

    if name == "skinny_swiglu":
        a = torch.randn(batch, hidden, device=device).bfloat16()
        w = weights(2 * width, hidden, 4)
        run = lambda i: ops.linear_swiglu(a, w[i % 4])
        work = f"{2 * width * hidden * 2 / 1e6:.1f} MB of weights"
    elif name == "skinny_down":
        a = torch.randn(batch, width, device=device).bfloat16()
        w = weights(hidden, width, 8)
        residual = torch.zeros(batch, hidden, device=device)
        run = lambda i: ops.linear_add(a, w[i % 8], None, residual)
        work = f"{hidden * width * 2 / 1e6:.1f} MB of weights"
    elif name == "decode_attention":
        ctx, view = batch_context([1] * batch, [context - 1] * batch)
        q = torch.randn(batch, heads, head_dim, device=device).bfloat16()
        run = lambda i: ops.paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                            scale=head_dim ** -0.5, window=None, ctx=ctx, view=view)
        work = f"{batch * context * 2 * kv_heads * head_dim * 2 / 1e6:.1f} MB of keys and values"
    elif name == "prefill_attention":
        ctx, view = batch_context([PREFILL_TOKENS], [0])
        q = torch.randn(PREFILL_TOKENS, heads, head_dim, device=device).bfloat16()
        run = lambda i: ops.paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                            scale=head_dim ** -0.5, window=None, ctx=ctx, view=view)
        work = f"{4 * heads * head_dim * PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2 / 1e9:.1f} GFLOP"
    elif name == "tcgen05_swiglu":
        a = torch.randn(PREFILL_TOKENS, hidden, device=device).bfloat16()
        w = weights(2 * width, hidden, 2)
        run = lambda i: ops.linear_swiglu(a, w[i % 2])
        work = f"{2 * PREFILL_TOKENS * 2 * width * hidden / 1e9:.1f} GFLOP"
    elif name == "sampling":
        vocab = LFM2_1_2B["vocab_size"]
        logits = [torch.randn(batch, vocab, device=device) * 3 for _ in range(4)]
        temperature = torch.full((batch,), 0.8, device=device)
        top_k = torch.full((batch,), 40, dtype=torch.int32, device=device)
        top_p = torch.full((batch,), 0.9, device=device)
        seed = torch.arange(batch, dtype=torch.int64, device=device)
        steps = torch.zeros(batch, dtype=torch.int32, device=device)
        run = lambda i: ops.sample(logits[i % 4], temperature, top_k, top_p, seed, steps)
        work = f"{batch} rows of {vocab} logits, temperature 0.8, top-k 40, top-p 0.9"
    else:
        print(f"unknown kernel case {name!r}")
        return 2
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(8):
        run(i)
    stop.record()
    torch.cuda.synchronize()
    ops.check_errors()
    print(json.dumps({"kernel": name, "us": round(start.elapsed_time(stop) * 1e3 / 8, 2),
                      "work": work, "batch": batch, "context": context}))
    return 0


def product_fractions(model, batch, peak):
    """The matrix products of the step alone, as the baseline's targets are stated for them:
    decode products against HBM bandwidth (bytes of weights / time), prefill products against
    the bf16 tensor peak. Each distinct product of the model is timed in a CUDA graph of
    back-to-back calls on several copies of its weights (so that none is found in L2)."""
    import torch

    ops, device = model.ops, "cuda:0"

    def graph_time(fn, copies, inner):
        for i in range(min(copies, 3)):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(inner):
                fn(i % copies)
        graph.replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(5):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / 1e3 / (5 * inner)

    # (weight, kind, how many times a step runs it); kind picks the epilogue the engine uses
    seen: dict = {}
    for block in model.layers:
        mixer, ffn = block.mixer, block.feed_forward
        first = getattr(mixer, "qkv", None)
        first = first if first is not None else mixer.in_proj
        last = getattr(mixer, "out", None)
        last = last if last is not None else mixer.out_proj
        for weight, kind in ((first, "plain"), (last, "add"), (ffn.gate_up, "swiglu"),
                             (ffn.down, "add")):
            key = (tuple(weight.shape), kind)
            seen.setdefault(key, [weight, 0])[1] += 1
    decode_bytes = decode_seconds = prefill_flops = prefill_seconds = 0.0
    for (shape, kind), (weight, count) in seen.items():
        n, k = shape
        copies = max(2, min(16, int(300e6 // (n * k * 2))))
        weights = [weight] + [torch.randn_like(weight) * 0.02 for _ in range(copies - 1)]
        for rows in (batch, PREFILL_TOKENS):
            a = torch.randn(rows, k, device=device).bfloat16()
            residual = torch.zeros(rows, n, device=device)
            if kind == "plain":
                fn = lambda i: ops.linear(a, weights[i])
            elif kind == "swiglu":
                fn = lambda i: ops.linear_swiglu(a, weights[i])
            else:
                fn = lambda i: ops.linear_add(a, weights[i], None, residual)
            seconds = graph_time(fn, copies, copies * (2 if rows == batch else 1))
            if rows == batch:
                decode_bytes += count * n * k * 2
                decode_seconds += count * seconds
            else:
                prefill_flops += count * 2.0 * rows * n * k
                prefill_seconds += count * seconds
        del weights
    return {"decode_products_gbs": round(decode_bytes / decode_seconds / 1e9, 1),
            "decode_products_hbm_frac": round(decode_bytes / decode_seconds / 1e9 / peak["hbm_gbs"], 4),
            "prefill_products_tflops": round(prefill_flops / prefill_seconds / 1e12, 1),
            "prefill_products_frac": round(prefill_flops / prefill_seconds / 1e12 / peak["bf16_tflops"], 4)}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--layers", type=int, default=LFM2_1_2B["num_hidden_layers"])
    parser.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    parser.add_argument("--kernel", default=None,
                        help="run one kernel alone instead of the benchmark: skinny_swiglu, "
                             "skinny_down, decode_attention, prefill_attention, tcgen05_swiglu, "
                             "sampling")
    parser.add_argument("--dependent-launches", type=int, default=1,
                        help="1: kernels of a decode step may start while the one before ends")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.kernel:
        return kernel_case(args.kernel, args.batch, args.context)
    warmup = max(args.warmup, 3)

    import torch

    peak = peaks()
    largest = 64 if not args.skip_points else args.batch
    engine = build_engine(LFM2_1_2B, args.layers, max(largest, args.batch), args.context,
                          warmup + args.steps)
    model, spec = engine.model, engine.model.spec
    model.ops.set_dependent_launches(bool(args.dependent_launches))
    weight_bytes = model.weight_bytes()
    kv_per_token = engine._bytes_per_token()
    state_bytes = sum(g.storage[:, 0].numel() * g.storage.element_size()
                      for g in engine.cache.states)

    launches_per_step = count_step_launches(engine, args.batch)
    sampler = ClockSampler()
    seconds, clocks, mean_context, _ = time_decode(engine, args.batch, args.context, warmup,
                                                   args.steps, seed=1, sampler=sampler)
    value = args.batch * args.steps / seconds
    step_bytes = weight_bytes + args.batch * (mean_context * kv_per_token + 2 * state_bytes)
    achieved = step_bytes / (seconds / args.steps) / 1e9

    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            s, _, _, _ = time_decode(engine, batch, args.context, warmup, args.steps, seed=2 + batch)
            points[f"decode_b{batch}"] = round(batch * args.steps / s, 1)

    e2e_seconds, h2d = time_e2e(engine, args.batch, args.context, warmup, args.steps, seed=7)
    e2e_value = args.batch * args.steps / e2e_seconds

    prefill_seconds = time_prefill(engine, PREFILL_TOKENS, 2, 3, seed=11)
    flops = model_flops(spec, PREFILL_TOKENS)
    products = None if args.skip_points else product_fractions(model, args.batch, peak)

    line = {
        "metric": "decode tok/s at batch 8 (LFM2-1.2B shape, bf16, context 4096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(seconds / args.steps * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), seeded uniform-random token ids",
        "config": {
            "model": "LFM2-1.2B shape", "layers": args.layers,
            "layers_full_model": LFM2_1_2B["num_hidden_layers"],
            "hidden": spec.hidden_size, "heads": LFM2_1_2B["num_attention_heads"],
            "kv_heads": LFM2_1_2B["num_key_value_heads"],
            "head_dim": spec.hidden_size // LFM2_1_2B["num_attention_heads"],
            "ffn_width": spec.layers[0].feed_forward["width"], "vocab": spec.vocab_size,
            "conv_taps": LFM2_1_2B["conv_L_cache"], "attention_layers":
                sum(1 for l in spec.layers if l.mixer.kind == "attention"),
            "global_batch": args.batch, "seq_len": args.context, "page_size": PAGE_SIZE,
            "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (2.3 GB of weights per step)",
            "peaks": peak["source"],
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                "ms_per_step": round(e2e_seconds / args.steps * 1e3, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches_per_step * args.steps,
        "launches_per_step": launches_per_step,
        "prefill": {"value": round(PREFILL_TOKENS / prefill_seconds, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_seconds * 1e3, 3),
                    "frac": round(flops / prefill_seconds / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4),
                     "bytes_per_step": int(step_bytes)},
        "points": points,
        "products": products,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
