"""The Python entry point: ``Engine`` with generate / stream / submit, in the manner of the
reference's ``Engine`` (src/mlx_one/engine/public.py:61-485) and text API
(src/mlx_one/text/generation.py:209-263).

Differences that the GPU design brings: requests are batched continuously by one scheduler
and run through one step function; the loop is driven by the caller's thread, or by a thread
of the engine's own with ``BatchingConfig(loop_thread=True)`` (the reference's actor thread);
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
from .scheduler import (PENDING, BatchingConfig, Phase, Request, RequestTimeoutError, Scheduler)


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
    flag_at: int = 0                  # where in ``host`` the kernels' error flag lies
    report: Any = None                # the device tensor being copied, kept until the copy is read


class EngineRequestHandle:
    """A submitted request.

    Without a loop thread (``BatchingConfig.loop_thread`` False, the default) nothing runs
    until somebody drives the loop: ``result()`` does (until this request is done), and so do
    ``Engine.step()``, ``Engine.run()``, ``generate*`` and the iterators of ``stream*``.
    ``done()`` alone only looks; polling it without one of those calls waits for ever. With a
    loop thread the engine drives itself and ``result()`` only waits."""

    def __init__(self, engine: "Engine", request: Request, prompt_text: str) -> None:
        self._engine = engine
        self.request = request
        self.prompt_text = prompt_text
        self.submitted_at = time.perf_counter()
        self.first_token_at: float | None = None
        self.finished_at: float | None = None
        self.stopped_text: str | None = None      # the text up to a stop string that matched

    def done(self) -> bool:
        return self.request.phase is Phase.FINISHED

    def cancel(self) -> None:
        with self._engine._turn:
            self._engine._scheduler.cancel(self.request)

    def result(self) -> GenerationResult:
        while not self.done():
            self._engine._drive_once()
        return self._engine._result(self)

    def tokens(self) -> Iterator[int]:
        """The request's tokens as they are committed (this handle's output queue): blocks,
        driving or waiting as ``result()`` does, until the request is done. A token that a
        later stop-string match takes back may have been handed out already."""
        sent = 0
        while True:
            if not self.done():
                self._engine._drive_once()
            finished = self.done()
            output = self.request.output
            while sent < len(output):
                sent += 1
                yield output[sent - 1]
            if finished:
                return


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
        self._copy_stream: Any = None
        self._inflight: _InFlight | None = None
        self._turn = threading.RLock()       # one thread at a time plans, launches and commits
        self._stepped = threading.Condition()   # notified after every turn
        self._wake = threading.Condition()      # the loop thread sleeps here while idle
        self._closing = False
        self._thread: threading.Thread | None = None
        if self.batching_config.loop_thread:
            self._thread = threading.Thread(target=self._loop, name="mlx-one_b200-loop",
                                            daemon=True)
            self._thread.start()

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

    @property
    def runner(self) -> Runner:
        """The step function that this engine drives (for replay, tests and measurements)."""
        return self._runner

    def cache_bytes_per_token(self) -> int:
        """Bytes of keys and values that one token of context holds, over all layers."""
        return self._bytes_per_token()

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
            options = options.replace(max_tokens=limit - len(prompt))
        with self._turn:
            request = Request(self._scheduler.new_id(), prompt, options,
                              eos_token_ids=self._loaded.spec.eos_token_ids)
            if options.stop and self._tokenizer is None:
                raise ValueError("stop strings are matched in text; this model folder has no "
                                 "tokenizer.json")
            self._scheduler.submit(request)
            handle = EngineRequestHandle(self, request, prompt_text)
            self._handles[request.request_id] = handle
        with self._wake:
            self._wake.notify_all()
        return handle

    def submit(self, prompt: str, options: TextGenerationOptions | None = None,
               **option_kwargs) -> EngineRequestHandle:
        """Queues a request and returns at once. See ``EngineRequestHandle`` for who drives
        the loop: without ``loop_thread`` the request makes no progress until a caller does."""
        return self.submit_ids(self.encode(prompt), self._options(options, option_kwargs),
                               prompt_text=prompt)

    # ------------------------------------------------------------------ the loop

    def step(self) -> list[Request]:
        """One scheduler turn. Returns the requests that got a token or finished.

        A step is planned, launched, its chosen tokens are copied to pinned host memory, and
        committed when that copy has landed. With ``pipeline_decode`` the next step (decodes,
        prompt portions, newly admitted requests) is launched before the last one is
        committed: a decode whose token is not known yet takes it on the device, where it was
        chosen, so the host's planning and bookkeeping run under the GPU's work. A request
        then learns of its end-of-sequence token one step late; the extra token computed for
        it is dropped.

        Turns exclude one another, so that several threads (``async_generate`` runs each
        request's wait on a thread of its own) may drive the loop: whichever holds the turn
        moves every running request on by one step."""
        with self._turn:
            touched = self._step()
        with self._stepped:
            self._stepped.notify_all()
        return touched

    def _loop(self) -> None:
        """The loop thread: turns while there is work, sleeps until a submit otherwise. A step
        that raises ends the requests it held (their ``result()`` raises the error); the
        thread goes on."""
        if self.model.runtime.device.type == "cuda":
            torch.cuda.set_device(self.model.runtime.device)
        while not self._closing:
            if self._scheduler.has_work() or self._inflight is not None:
                try:
                    self.step()
                except BaseException as error:          # noqa: BLE001
                    with self._turn:
                        self._abandon(error)
                    with self._stepped:
                        self._stepped.notify_all()
            else:
                with self._wake:
                    if not (self._closing or self._scheduler.has_work()):
                        self._wake.wait(0.05)

    def _abandon(self, error: BaseException) -> None:
        """After a step that raised: nothing in flight is trusted, every running request ends
        with ``error``."""
        self._inflight = None
        self._scheduler.fail(list(self._scheduler.running), error)

    def _drive_once(self) -> None:
        """One turn of the loop if no other thread is in one; else a wait until that thread's
        turn has ended. A thread that waits for its request thus sees it finish without having
        to win the lock from the thread that keeps the loop going. With a loop thread the
        caller never drives."""
        if self._thread is not None:
            with self._stepped:
                self._stepped.wait(0.005)
            return
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
        """Plans and launches the next step, then commits the step that was in flight. The
        scheduler is told of a launch at once (``advance``: prompts move on, drawn tokens count
        as pending), so the next step can be planned while the tokens of the last one are still
        on their way; a decode whose token is pending takes it on the device."""
        previous = self._inflight
        launched = None
        if previous is None or self._may_run_ahead():
            planned = self._scheduler.plan()
            if planned:
                launched = self._launch(planned, ahead=previous is not None)
                self._scheduler.advance(planned)
        self._inflight = launched          # (a kernel fault found in `previous` drops it too)
        touched = self._finish(previous) if previous is not None else []
        launched = self._inflight
        if launched is not None and not self.batching_config.pipeline_decode:
            self._inflight = None
            touched += self._finish(launched)
        return touched

    def _may_run_ahead(self) -> bool:
        """Whether the next step may be planned before the tokens of the step in flight are
        known: not while a running request has stop strings, whose match must end the request
        before anything else is run for it."""
        if not self.batching_config.pipeline_decode:
            return False
        return not any(r.options.stop for r in self._scheduler.running)

    def _launch(self, planned, ahead: bool = False) -> "_InFlight":
        """Launches a step; the tokens of the requests that draw one are chosen on the device
        inside it (argmax, or the sampling kernel with each request's options, seed and count
        of tokens drawn so far, pending ones included)."""
        started = time.perf_counter()
        entries = []
        for item in planned:
            want = (len(item.tokens) - 1,) if item.samples else ()
            if item.tokens[0] == PENDING:
                entries.append(StepEntry(item.request.request_id, (0,), want, from_device=True))
            else:
                entries.append(StepEntry(item.request.request_id, item.tokens, want))
        drawing = [item.request for item in planned if item.samples]
        greedy = bool(drawing) and all(r.options.temperature == 0 for r in drawing)
        draw = None
        if drawing and not greedy:
            draw = [(r.options.temperature, r.options.top_k or 0, r.options.top_p, r.options.seed,
                     len(r.output) + r.pending) for r in drawing]
        self._runner.step(entries, greedy=greedy, draw=draw)
        host = event = None
        flag_at = 0
        if drawing:
            report = self._runner.last_report
            flag_at = report.numel() - 1
            host, event = self._start_copy(report)
        self._stats["steps"] += 1
        self._stats["steps_ahead"] += 1 if ahead else 0
        self._stats["tokens_run"] += sum(len(item.tokens) for item in planned)
        prompt_tokens = sum(len(item.tokens) for item in planned
                            if item.request.phase is Phase.PREFILL)
        return _InFlight(list(planned), host, event, len(drawing), bool(drawing),
                         launched_at=started, ahead=ahead, prompt_tokens=prompt_tokens,
                         flag_at=flag_at, report=report if drawing else None)

    def _finish(self, inflight: "_InFlight") -> list[Request]:
        sampled: list[int] = []
        if inflight.host is not None:
            if inflight.event is not None:
                inflight.event.synchronize()
            sampled = inflight.host[:inflight.draws].tolist()
            code = int(inflight.host[inflight.flag_at])    # the kernels' error flag, same copy
            if code:
                return self._kernel_fault(code, inflight)
        planned = inflight.planned
        # (a request that has ended since this step was launched drops its token there)
        touched = self._scheduler.resolve(planned, sampled, stop_at=self._stop_at)
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

    def _kernel_fault(self, code: int, inflight: "_InFlight") -> list[Request]:
        """A kernel of this step (or of one before it whose tokens were not read) set the
        device's error flag: a wait that gave up, a key without a page, a token outside the
        vocabulary. Its tokens are not committed; the step's requests and those of a step
        launched ahead end with a ``KernelError`` and give their pages back."""
        ops = self.model.ops
        requests = [item.request for item in inflight.planned]
        ahead = self._inflight
        if ahead is not None and ahead is not inflight:
            if ahead.event is not None:
                ahead.event.synchronize()
            requests += [item.request for item in ahead.planned]
        self._inflight = None
        ops.error_flag.zero_()
        error = getattr(ops, "describe_error", lambda c: RuntimeError(f"kernel error {c}"))(code)
        failed = list({id(r): r for r in requests if r.phase is not Phase.FINISHED}.values())
        self._scheduler.fail(failed, error)
        self._stats["kernel_faults"] = self._stats.get("kernel_faults", 0) + 1
        now = time.perf_counter()
        for request in failed:
            handle = self._handles.get(request.request_id)
            if handle is not None:
                handle.finished_at = now
        return failed

    def _stop_at(self, request: Request, token: int) -> int | None:
        """Whether the text of ``request`` with ``token`` appended contains one of its stop
        strings; if so, how many of its tokens lie wholly before the match. The reference ends
        a request on a stop string wherever its text is produced
        (src/mlx_one/text/generation.py:266-290, 682-697)."""
        tokens = request.output + [token]
        text = self.decode(tokens)
        cut, matched = self._apply_stop(text, request.options.stop)
        if not matched:
            return None
        keep = 0
        while keep < len(request.output) and len(self.decode(tokens[:keep + 1])) <= len(cut):
            keep += 1
        handle = self._handles.get(request.request_id)
        if handle is not None:
            handle.stopped_text = cut
        return keep

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
            "committed_at": committed_at,
        }
        self._stats["steps_committed"] += 1
        self._traces.append(record)
        if self._trace_sink is not None:
            self._trace_sink(record)

    def set_trace_sink(self, sink) -> None:
        """``sink(record)`` is called with every committed step's record from now on (None:
        nobody)."""
        self._trace_sink = sink

    def step_traces(self) -> list[dict[str, Any]]:
        """The records of the last steps (at most 4096), oldest first."""
        return list(self._traces)

    def _start_copy(self, report: torch.Tensor):
        """Starts the copy of a step's report to the host: the chosen tokens and, behind them,
        the kernels' error flag as it stood at the end of the step, so that a fault is seen
        with the tokens it spoilt and costs neither a copy nor a wait of its own. Returns (host
        buffer, event); the flag is the buffer's last copied entry."""
        count = report.numel()
        if report.device.type != "cuda":
            return report.clone(), None
        self._copy_turn ^= 1
        buffer = self._pinned[self._copy_turn]
        if buffer is None or buffer.numel() < count:
            buffer = torch.zeros(max(count, 256), dtype=torch.int32, pin_memory=True)
            self._pinned[self._copy_turn] = buffer
        # On a stream of its own, behind the step: the next step's metadata copy (host to device)
        # then does not queue behind this one (device to host), and its kernels, which will
        # overwrite the report at their end, wait for this copy only after their own copy.
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=report.device)
        main = torch.cuda.current_stream(report.device)
        stepped = torch.cuda.Event()
        stepped.record(main)
        self._copy_stream.wait_event(stepped)
        with torch.cuda.stream(self._copy_stream):
            buffer[:count].copy_(report, non_blocking=True)
            event = torch.cuda.Event()
            event.record(self._copy_stream)
        self._runner.wait_before_kernels = event
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
        if request.finish_reason == "error":
            raise request.error or RuntimeError("the request's step failed")
        finished = handle.finished_at or time.perf_counter()
        first = handle.first_token_at or finished
        count = len(request.output)
        timings = {"total_s": finished - handle.submitted_at,
                   "time_to_first_token_s": first - handle.submitted_at}
        if count > 1 and finished > first:
            # decoding speed leaves out the prompt and the first token, as the reference does
            timings["decode_tokens_per_s"] = (count - 1) / (finished - first)
        reason = request.finish_reason or "length"
        text = (handle.stopped_text if handle.stopped_text is not None
                else self.decode(request.output))
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
        """Chunks of a request as its tokens are committed. With stop strings, text that may
        still turn into one is held back; when one matches (seen where the token is committed,
        so the request has ended and freed its pages already) the last chunk brings the text up
        to the match."""
        request, sent, text_sent = handle.request, 0, ""
        stop = request.options.stop
        while True:
            if not handle.done():
                self._drive_once()
            finished = handle.done()
            output = list(request.output)
            while sent < len(output):
                sent += 1
                piece = ""
                if self._tokenizer is not None:
                    text = self.decode(output[:sent])
                    if stop and not (finished and sent == len(output)):
                        text = self._hold_back(text, stop)
                    if len(text) > len(text_sent):
                        piece, text_sent = text[len(text_sent):], text
                yield GenerationChunk(output[sent - 1], piece, sent)
            if finished:
                self._handles.pop(request.request_id, None)
                reason = request.finish_reason or "length"
                if reason == "timeout":
                    raise RequestTimeoutError("generation request timed out")
                if reason == "error":
                    raise request.error or RuntimeError("the request's step failed")
                trailing = ""
                if handle.stopped_text is not None and len(handle.stopped_text) > len(text_sent):
                    trailing = handle.stopped_text[len(text_sent):]
                yield GenerationChunk(None, trailing, len(request.output),
                                      "stop" if reason == "cancelled" else reason,
                                      request.terminal_token_id)
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
        return {**self._stats, **self._runner.graph_stats(),
                "waiting": len(self._scheduler.waiting),
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
        """Ends every request, gives all pages back and stops the loop thread. Raises the
        ``KernelError`` of a fault that the device's error flag still holds, after cleaning
        up."""
        self._closing = True
        with self._wake:
            self._wake.notify_all()
        if self._thread is not None and self._thread is not threading.current_thread():
            self._thread.join(timeout=30)
        self._thread = None
        with self._turn:
            if self._inflight is not None:
                inflight, self._inflight = self._inflight, None
                self._finish(inflight)
            for request in list(self._scheduler.running) + list(self._scheduler.waiting):
                self._scheduler.cancel(request)
            self._scheduler.plan()
            self._cache.close_all()
        with self._stepped:
            self._stepped.notify_all()
        self.model.ops.check_errors()

    def __enter__(self) -> "Engine":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
