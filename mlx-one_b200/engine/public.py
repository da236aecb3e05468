"""The Python entry point: ``Engine`` with generate / stream / submit, in the manner of the
reference's ``Engine`` (src/mlx_one/engine/public.py:61-485) and text API
(src/mlx_one/text/generation.py:209-263).

Differences that the GPU design brings: requests are batched continuously by one scheduler
and run through one step function, the caller's thread drives the loop (no actor thread),
and there are entry points that take and return token ids, because a model with random
weights has no tokenizer.
"""

from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Iterator, Sequence

import torch

from ..cache.manager import CacheManager
from ..sampling.options import GenerationChunk, GenerationResult, TextGenerationOptions
from .loading import LoadedModel, load_model
from .runner import Runner, StepEntry
from .scheduler import (BatchingConfig, Phase, Request, RequestTimeoutError, Scheduled,
                        Scheduler)


@dataclass(frozen=True)
class CacheConfig:
    """``block_size_tokens``: tokens per page (the reference's name,
    src/mlx_one/engine/cache_specs.py:174-204). The pool's size is ``capacity_tokens`` if
    given, else what ``memory_budget_bytes`` buys, else 64 * 1024 tokens."""

    block_size_tokens: int = 16
    capacity_tokens: int | None = None
    memory_budget_bytes: int | None = None
    max_requests: int | None = None

    def __post_init__(self) -> None:
        if self.block_size_tokens not in (1, 2, 4, 8, 16, 32, 64, 128):
            raise ValueError("cache block size must be a power of two up to 128")
        for name in ("capacity_tokens", "memory_budget_bytes", "max_requests"):
            value = getattr(self, name)
            if value is not None and value < 1:
                raise ValueError(f"{name} must be positive")


@dataclass
class _InFlight:
    """A launched step whose chosen tokens are on their way to the host."""

    planned: list
    host: Any
    event: Any
    draws: int
    chosen_on_device: bool
    launched_at: float = 0.0
    ahead: bool = False
    prompt_tokens: int = 0


class EngineRequestHandle:
    """A submitted request. ``result()`` drives the engine until the request is done."""

    def __init__(self, engine: "Engine", request: Request, prompt_text: str) -> None:
        self._engine = engine
        self.request = request
        self.prompt_text = prompt_text
        self.submitted_at = time.perf_counter()
        self.first_token_at: float | None = None
        self.finished_at: float | None = None

    def done(self) -> bool:
        return self.request.phase is Phase.FINISHED

    def cancel(self) -> None:
        with self._engine._turn:
            self._engine._scheduler.cancel(self.request)

    def result(self) -> GenerationResult:
        while not self.done():
            self._engine._drive_once()
        return self._engine._result(self)


class Engine:
    def __init__(self, model: str | Path | LoadedModel, *, cache_config: CacheConfig | None = None,
                 batching_config: BatchingConfig | None = None,
                 execution_dtype: str | None = None, device: str = "cuda:0",
                 ops: Any = None, revision: str | None = None, offline: bool = True,
                 cache_dir: str | Path | None = None,
                 tokenizer_source: str | Path | None = None,
                 trace_sink: Any = None) -> None:
        """``model``: a model folder (config.json + safetensors) or a loaded model.
        ``execution_dtype``: "bfloat16" (default) or "float32" (everything in true 32-bit).
        ``revision``, ``offline``, ``cache_dir``: the reference's names for fetching a model by
        its hub id (src/mlx_one/engine/public.py:64-85). This engine loads local folders only:
        they are accepted for a local folder (a revision must then be None) and a name that is
        no folder is refused. ``tokenizer_source``: a folder with ``tokenizer.json``, or the
        file, when it is not in the model folder. ``trace_sink``: called with the record of
        every committed step (see ``step_traces``)."""
        if not isinstance(model, LoadedModel):
            if revision is not None:
                raise ValueError("revision names a hub snapshot; this engine loads local folders")
            if not Path(model).is_dir():
                raise FileNotFoundError(
                    f"{model!s} is no model folder; models are not fetched by name "
                    f"(offline={offline}, cache_dir={cache_dir})")
        self._tokenizer_source = None if tokenizer_source is None else Path(tokenizer_source)
        self._loaded = model if isinstance(model, LoadedModel) else load_model(
            model, execution_dtype or "bfloat16", device, ops)
        built = self._loaded.model
        self.cache_config = cache_config or CacheConfig()
        self.batching_config = batching_config or BatchingConfig()
        capacity = self.cache_config.capacity_tokens
        if capacity is None and self.cache_config.memory_budget_bytes is not None:
            capacity = max(self.cache_config.memory_budget_bytes // self._bytes_per_token(), 1)
        if capacity is None:
            capacity = 64 * 1024
        max_requests = self.cache_config.max_requests or max(self.batching_config.max_sequences, 1)
        self._cache = CacheManager(
            built.cache_needs, page_size=self.cache_config.block_size_tokens,
            capacity_tokens=capacity, max_requests=max_requests, dtype=built.runtime.dtype,
            device=built.runtime.device,
            max_step_tokens=self.batching_config.max_scheduled_tokens)
        self._runner = Runner(built, self._cache)
        self._scheduler = Scheduler(self.batching_config, self._cache)
        self._handles: dict[Any, EngineRequestHandle] = {}
        self._tokenizer = self._load_tokenizer()
        self._stats = {"steps": 0, "steps_ahead": 0, "steps_committed": 0, "tokens_run": 0,
                       "tokens_sampled": 0}
        self._traces: deque[dict[str, Any]] = deque(maxlen=4096)
        self._trace_sink = trace_sink          # called with every step's record, if given
        self._pinned: list[torch.Tensor | None] = [None, None]
        self._copy_turn = 0
        self._inflight: _InFlight | None = None
        self._turn = threading.RLock()       # one thread at a time plans, launches and commits
        self._stepped = threading.Condition()   # notified after every turn

    # ------------------------------------------------------------------ set-up

    def _bytes_per_token(self) -> int:
        from ..parts.base import PagedKeyValues

        size = torch.empty((), dtype=self._loaded.model.runtime.dtype).element_size()
        total = sum(2 * need.kv_heads * need.head_dim * size
                    for need in self._loaded.model.cache_needs.values()
                    if isinstance(need, PagedKeyValues))
        return max(total, 1)

    def _load_tokenizer(self):
        path = self._loaded.path / "tokenizer.json" if self._loaded.path else None
        if self._tokenizer_source is not None:
            source = self._tokenizer_source
            path = source / "tokenizer.json" if source.is_dir() else source
            if not path.is_file():
                raise FileNotFoundError(f"tokenizer_source: {path} does not exist")
        if path is None or not path.is_file():
            return None
        from tokenizers import Tokenizer

        return Tokenizer.from_file(str(path))

    @property
    def model(self):
        return self._loaded.model

    @property
    def cache(self) -> CacheManager:
        return self._cache

    # ------------------------------------------------------------------ text <-> ids

    def encode(self, prompt: str) -> list[int]:
        """Prompt text -> token ids, with a BOS token in front if the tokenizer did not put
        one there (the reference's rule for LFM2, src/mlx_one/text/prompts.py:6-17)."""
        if self._tokenizer is None:
            raise ValueError("this model folder has no tokenizer.json; pass token ids "
                             "(generate_ids) instead of text")
        ids = list(self._tokenizer.encode(prompt).ids)
        bos = self._loaded.spec.bos_token_id
        if bos is not None and (not ids or ids[0] != bos):
            ids.insert(0, bos)
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        if self._tokenizer is None:
            return ""
        return self._tokenizer.decode(list(ids))

    # ------------------------------------------------------------------ requests

    def _options(self, options, kwargs) -> TextGenerationOptions:
        if options is not None and kwargs:
            raise ValueError("pass options or option keywords, not both")
        return options if options is not None else TextGenerationOptions(**kwargs)

    def submit_ids(self, prompt_ids: Sequence[int], options: TextGenerationOptions | None = None,
                   *, prompt_text: str = "", **option_kwargs) -> EngineRequestHandle:
        options = self._options(options, option_kwargs)
        prompt = tuple(int(t) for t in prompt_ids)
        limit = self._loaded.spec.max_positions
        if len(prompt) >= limit:
            raise ValueError(f"prompt of {len(prompt)} tokens reaches the model's {limit} positions")
        if len(prompt) + options.max_tokens > limit:
            options = TextGenerationOptions(**{**options.__dict__,
                                               "max_tokens": limit - len(prompt)})
        with self._turn:
            request = Request(self._scheduler.new_id(), prompt, options,
                              eos_token_ids=self._loaded.spec.eos_token_ids)
            self._scheduler.submit(request)
            handle = EngineRequestHandle(self, request, prompt_text)
            self._handles[request.request_id] = handle
        return handle

    def submit(self, prompt: str, options: TextGenerationOptions | None = None,
               **option_kwargs) -> EngineRequestHandle:
        return self.submit_ids(self.encode(prompt), self._options(options, option_kwargs),
                               prompt_text=prompt)

    # ------------------------------------------------------------------ the loop

    def step(self) -> list[Request]:
        """One scheduler turn. Returns the requests that got a token or finished.

        A step is planned, launched, its chosen tokens are copied to pinned host memory, and
        committed when that copy has landed. While every running request decodes
        (``pipeline_decode``), the next step is launched before the last one is committed: its
        input tokens are the ones the device has just chosen, so the host's bookkeeping runs
        under the GPU's work. A request then learns of its end-of-sequence token one step
        late; the extra token computed for it is dropped.

        Turns exclude one another, so that several threads (``async_generate`` runs each
        request's wait on a thread of its own) may drive the loop: whichever holds the turn
        moves every running request on by one step."""
        with self._turn:
            touched = self._step()
        with self._stepped:
            self._stepped.notify_all()
        return touched

    def _drive_once(self) -> None:
        """One turn of the loop if no other thread is in one; else a wait until that thread's
        turn has ended. A thread that waits for its request thus sees it finish without having
        to win the lock from the thread that keeps the loop going."""
        if self._turn.acquire(blocking=False):
            try:
                self._step()
            finally:
                self._turn.release()
            with self._stepped:
                self._stepped.notify_all()
        else:
            with self._stepped:
                self._stepped.wait(0.005)

    def _step(self) -> list[Request]:
        previous = self._inflight
        if previous is not None:
            ahead = self._launch_ahead(previous)
            touched = self._finish(previous)
            self._inflight = ahead
            return touched
        planned = self._scheduler.plan()
        if not planned:
            return []
        launched = self._launch(planned)
        if self.batching_config.pipeline_decode and launched.chosen_on_device:
            self._inflight = launched
            return []
        return self._finish(launched)

    def _launch(self, planned, entries=None, ahead: int = 0) -> "_InFlight":
        """Launches a step; the tokens of the requests that draw one are chosen on the device
        inside it (argmax, or the sampling kernel with each request's options, seed and count
        of tokens drawn so far; ``ahead``: tokens drawn but not yet committed)."""
        started = time.perf_counter()
        if entries is None:
            entries = [StepEntry(item.request.request_id, item.tokens,
                                 (len(item.tokens) - 1,) if item.samples else ())
                       for item in planned]
        drawing = [item.request for item in planned if item.samples]
        greedy = bool(drawing) and all(r.options.temperature == 0 for r in drawing)
        draw = None
        if drawing and not greedy:
            draw = [(r.options.temperature, r.options.top_k or 0, r.options.top_p, r.options.seed,
                     len(r.output) + ahead) for r in drawing]
        self._runner.step(entries, greedy=greedy, draw=draw)
        host = event = None
        if drawing:
            host, event = self._start_copy(self._runner.last_greedy)
        self._stats["steps"] += 1
        self._stats["tokens_run"] += sum(len(item.tokens) for item in planned)
        # a step launched ahead holds decode tokens only (a request whose last portion is not
        # committed yet still counts as being in its prompt)
        prompt_tokens = 0 if ahead else sum(len(item.tokens) for item in planned
                                            if item.request.phase is Phase.PREFILL)
        return _InFlight(list(planned), host, event, len(drawing), bool(drawing),
                         launched_at=started, ahead=ahead > 0, prompt_tokens=prompt_tokens)

    def _launch_ahead(self, previous: "_InFlight"):
        """The step after ``previous``, launched before ``previous`` is committed, or None if
        it cannot be known yet what that step will be."""
        scheduler = self._scheduler
        if not (self.batching_config.pipeline_decode and previous.chosen_on_device) or scheduler.waiting:
            return None
        drew = {id(item.request) for item in previous.planned if item.samples}
        running = scheduler.running
        if any(id(r) not in drew or r.cancelled or r.options.stop for r in running):
            return None          # a prompt still in portions, decodes taking turns, a cancel
        now = scheduler.clock()
        if any(r.deadline is not None and now >= r.deadline for r in running):
            return None          # a request's time is up: the next plan ends it
        going_on = [r for r in running if len(r.output) + 1 < r.options.max_tokens]
        if not going_on or len(going_on) > self.batching_config.max_scheduled_tokens:
            return None
        planned = [Scheduled(r, (0,), True) for r in going_on]
        entries = [StepEntry(r.request_id, (0,), (0,), from_device=True) for r in going_on]
        self._stats["steps_ahead"] += 1
        return self._launch(planned, entries, ahead=1)

    def _finish(self, inflight: "_InFlight") -> list[Request]:
        sampled: list[int] = []
        if inflight.host is not None:
            if inflight.event is not None:
                inflight.event.synchronize()
            sampled = inflight.host[:inflight.draws].tolist()
        planned = inflight.planned
        if any(item.request.phase is Phase.FINISHED for item in planned):
            # launched ahead for a request that has ended meanwhile: its token is dropped
            kept, tokens, drawn = [], [], iter(sampled)
            for item in planned:
                token = next(drawn) if item.samples else None
                if item.request.phase is Phase.FINISHED:
                    continue
                kept.append(item)
                if item.samples:
                    tokens.append(token)
            planned, sampled = kept, tokens
        touched = self._scheduler.commit(planned, sampled)
        now = time.perf_counter()
        self._trace(inflight, now)
        for request in touched:
            handle = self._handles.get(request.request_id)
            if handle is None:
                continue
            if handle.first_token_at is None:
                handle.first_token_at = now
            if request.phase is Phase.FINISHED:
                handle.finished_at = now
        self._stats["tokens_sampled"] += len(sampled)
        return touched

    def _trace(self, inflight: "_InFlight", committed_at: float) -> None:
        """One record per step, as the reference's runners keep them
        (src/mlx_one/engine/hybrid.py:242-251, kept in a deque of 4096 and handed to an optional
        sink, src/mlx_one/engine/actor.py:77,481-500). Nothing is padded here, so the tokens are
        the real ones; the duration is the host's, from the launch to the commit."""
        items = inflight.planned
        prompt_tokens = inflight.prompt_tokens
        tokens = sum(len(item.tokens) for item in items)
        record = {
            "step": self._stats["steps_committed"],
            "phase": "decode" if prompt_tokens == 0 else "prefill" if prompt_tokens == tokens
                     else "mixed",
            "request_ids": tuple(item.request.request_id for item in items),
            "batch_size": len(items), "tokens": tokens, "prompt_tokens": prompt_tokens,
            "decode_tokens": tokens - prompt_tokens, "draws": inflight.draws,
            "launched_ahead": inflight.ahead,
            "duration_s": committed_at - inflight.launched_at,
        }
        self._stats["steps_committed"] += 1
        self._traces.append(record)
        if self._trace_sink is not None:
            self._trace_sink(record)

    def step_traces(self) -> list[dict[str, Any]]:
        """The records of the last steps (at most 4096), oldest first."""
        return list(self._traces)

    def _start_copy(self, tokens: torch.Tensor):
        """Starts the copy of the chosen tokens to the host; returns (host buffer, event)."""
        if tokens.device.type != "cuda":
            return tokens.clone(), None
        self._copy_turn ^= 1
        buffer = self._pinned[self._copy_turn]
        if buffer is None or buffer.numel() < tokens.numel():
            buffer = torch.empty(max(tokens.numel(), 256), dtype=torch.int32, pin_memory=True)
            self._pinned[self._copy_turn] = buffer
        buffer[:tokens.numel()].copy_(tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return buffer, event

    def run(self) -> None:
        """Drives the loop until no request is waiting or running."""
        while self._scheduler.has_work() or self._inflight is not None:
            self.step()

    # ------------------------------------------------------------------ results

    def _result(self, handle: EngineRequestHandle) -> GenerationResult:
        request = handle.request
        self._handles.pop(request.request_id, None)
        if request.finish_reason == "timeout":
            raise RequestTimeoutError("generation request timed out")
        finished = handle.finished_at or time.perf_counter()
        first = handle.first_token_at or finished
        count = len(request.output)
        timings = {"total_s": finished - handle.submitted_at,
                   "time_to_first_token_s": first - handle.submitted_at}
        if count > 1 and finished > first:
            # decoding speed leaves out the prompt and the first token, as the reference does
            timings["decode_tokens_per_s"] = (count - 1) / (finished - first)
        reason = request.finish_reason or "length"
        text = self._apply_stop(self.decode(request.output), request.options.stop)[0]
        return GenerationResult(
            prompt=handle.prompt_text, text=text, prompt_tokens=len(request.prompt),
            generation_tokens=count, finish_reason="stop" if reason == "cancelled" else reason,
            model=str(self._loaded.path), timings=timings, token_ids=tuple(request.output))

    @staticmethod
    def _apply_stop(text: str, stop: Sequence[str]) -> tuple[str, bool]:
        cut = min((text.find(s) for s in stop if s in text), default=-1)
        return (text, False) if cut < 0 else (text[:cut], True)

    def generate_ids(self, prompt_ids: Sequence[int], options: TextGenerationOptions | None = None,
                     **option_kwargs) -> GenerationResult:
        return self.submit_ids(prompt_ids, self._options(options, option_kwargs)).result()

    def generate_batch_ids(self, prompts: Sequence[Sequence[int]],
                           options: TextGenerationOptions | Sequence[TextGenerationOptions]
                           | None = None) -> list[GenerationResult]:
        """Submits all prompts (waiting for queue room as needed) and runs them together."""
        many = list(options) if isinstance(options, (list, tuple)) else [options] * len(prompts)
        handles = []
        for prompt, option in zip(prompts, many):
            while len(self._scheduler.waiting) >= self.batching_config.queue_size:
                self.step()
            handles.append(self.submit_ids(prompt, option))
        self.run()
        return [handle.result() for handle in handles]

    def generate(self, prompt: str, options: TextGenerationOptions | None = None,
                 **option_kwargs) -> GenerationResult:
        return self.submit(prompt, self._options(options, option_kwargs)).result()

    async def async_generate_ids(self, prompt_ids: Sequence[int],
                                 options: TextGenerationOptions | None = None,
                                 **option_kwargs) -> GenerationResult:
        """``generate_ids`` for coroutines: the request is submitted at once and awaited on a
        worker thread that drives the loop, so requests of several coroutines are batched
        together. A cancelled coroutine cancels its request."""
        import asyncio

        handle = self.submit_ids(prompt_ids, options, **option_kwargs)
        try:
            return await asyncio.get_running_loop().run_in_executor(None, handle.result)
        except asyncio.CancelledError:
            handle.cancel()
            raise

    async def async_generate(self, prompt: str, *, options: TextGenerationOptions | None = None,
                             **option_kwargs) -> GenerationResult:
        """As the reference's ``Engine.async_generate`` (src/mlx_one/engine/public.py:412-424)."""
        return await self.async_generate_ids(self.encode(prompt),
                                             self._options(options, option_kwargs),
                                             prompt_text=prompt)

    def stream_ids(self, prompt_ids: Sequence[int], options: TextGenerationOptions | None = None,
                   **option_kwargs) -> Iterator[GenerationChunk]:
        handle = self.submit_ids(prompt_ids, self._options(options, option_kwargs))
        yield from self._stream(handle)

    def stream(self, prompt: str, options: TextGenerationOptions | None = None,
               **option_kwargs) -> Iterator[GenerationChunk]:
        handle = self.submit(prompt, self._options(options, option_kwargs))
        yield from self._stream(handle)

    def _stream(self, handle: EngineRequestHandle) -> Iterator[GenerationChunk]:
        request, sent, text_sent = handle.request, 0, ""
        stop = request.options.stop
        while True:
            if not handle.done():
                self._drive_once()
            while sent < len(request.output):
                sent += 1
                piece = ""
                if self._tokenizer is not None:
                    text, matched = self._apply_stop(self.decode(request.output[:sent]), stop)
                    # hold back text that may still turn into a stop string
                    safe = text if matched or handle.done() else self._hold_back(text, stop)
                    piece, text_sent = safe[len(text_sent):], max(safe, text_sent, key=len)
                    if matched:
                        with self._turn:
                            self._scheduler.finish(request, "stop")
                        yield GenerationChunk(request.output[sent - 1], piece, sent, "stop")
                        self._handles.pop(request.request_id, None)
                        return
                yield GenerationChunk(request.output[sent - 1], piece, sent)
            if handle.done():
                reason = request.finish_reason or "length"
                if reason == "timeout":
                    self._handles.pop(request.request_id, None)
                    raise RequestTimeoutError("generation request timed out")
                yield GenerationChunk(None, "", sent, "stop" if reason == "cancelled" else reason,
                                      request.terminal_token_id)
                self._handles.pop(request.request_id, None)
                return

    @staticmethod
    def _hold_back(text: str, stop: Sequence[str]) -> str:
        keep = 0
        for s in stop:
            for size in range(min(len(s) - 1, len(text)), 0, -1):
                if text.endswith(s[:size]):
                    keep = max(keep, size)
                    break
        return text[:len(text) - keep] if keep else text

    # ------------------------------------------------------------------ introspection

    def runtime_stats(self) -> dict[str, Any]:
        cache = self._cache.stats()
        return {**self._stats, "waiting": len(self._scheduler.waiting),
                "running": len(self._scheduler.running), "pages_total": cache.pages_total,
                "pages_free": cache.pages_free, "pages_low_water": cache.pages_low_water,
                "slots_free": cache.slots_free, "kernel_launches": self.model.ops.launches}

    def capabilities(self) -> dict[str, Any]:
        return {"architecture": self._loaded.spec.architecture,
                "dtype": str(self.model.runtime.dtype).replace("torch.", ""),
                "mixed_prefill_decode": True, "paged_cache": True,
                "page_size": self.cache_config.block_size_tokens,
                "capacity_tokens": self._cache.capacity_tokens,
                "max_sequences": self.batching_config.max_sequences,
                "sampling": ["greedy", "temperature", "top_k", "top_p", "seed"]}

    def close(self) -> None:
        if self._inflight is not None:
            self._finish(self._inflight)
            self._inflight = None
        for request in list(self._scheduler.running) + list(self._scheduler.waiting):
            self._scheduler.cancel(request)
        self._scheduler.plan()
        self._cache.close_all()

    def __enter__(self) -> "Engine":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
