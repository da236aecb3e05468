"""The scheduler above the step function: admits requests, cuts prompts into portions under
a token budget, decodes, finishes and frees. Host-only; it never touches a tensor.

Decisions:

* Admission is by reservation of a request's whole future (prompt + max_tokens), as in the
  reference (src/mlx_one/text/generation.py:114-123, src/mlx_one/engine/cache_manager.py:
  283-341). A request that could never fit is rejected when it is submitted; one that does
  not fit now waits. So pages cannot run out in the middle of a request, and nothing is ever
  preempted or recomputed. The waiting queue is served oldest first, but a request that does
  not fit now does not block a younger one that does.
* A step holds every running decode (one token each), then prompt portions of the running
  requests, oldest first, each at most ``prefill_chunk_size`` tokens, all prompt tokens
  together at most ``max_prefill_tokens``, everything together at most
  ``max_scheduled_tokens``. The reference's BatchScheduler chooses under the same three
  limits (src/mlx_one/engine/batching.py:81-117) but runs decodes and prompts as separate
  forwards; here they are one batch. If decodes alone exceed the budget they take turns, and
  room for a portion of the oldest prompt is always kept, so prompts cannot starve.
"""

from __future__ import annotations

import enum
import itertools
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Sequence

from ..cache.errors import CacheCapacityError
from ..cache.manager import CacheManager
from ..sampling.options import TextGenerationOptions


@dataclass(frozen=True)
class BatchingConfig:
    """Names and defaults of the reference's BatchingConfig (src/mlx_one/engine/batching.py:
    24-46), for the options that this scheduler has."""

    max_sequences: int = 1
    queue_size: int = 8
    prefill_chunk_size: int = 512
    max_scheduled_tokens: int = 2048
    max_prefill_tokens: int = 1024
    # seconds from its submission after which a request that has not finished is ended with
    # RequestTimeoutError; 0: never
    timeout: float = 600.0
    # not in the reference: launch the next step (the tokens that the step before it has just
    # chosen are taken on the device, where they were chosen) before that step's tokens have been
    # read back, so that the host's planning and bookkeeping run under the GPU's work
    pipeline_decode: bool = True
    # True: the engine owns a thread that drives the loop while requests are waiting or running,
    # as the reference's actor thread does (src/mlx_one/engine/actor.py:402-525); callers then
    # only wait. False: whoever waits for a request drives the loop from its own thread
    loop_thread: bool = False

    def __post_init__(self) -> None:
        for name in ("max_sequences", "queue_size", "prefill_chunk_size",
                     "max_scheduled_tokens", "max_prefill_tokens"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, int) or value < 1:
                raise ValueError(f"{name} must be positive")
        if isinstance(self.timeout, bool) or not isinstance(self.timeout, (int, float)) \
                or self.timeout < 0:
            raise ValueError("timeout must be zero or positive")


class QueueFullError(RuntimeError):
    """More requests are waiting than ``queue_size`` allows."""


class RequestTimeoutError(RuntimeError):
    """A request did not finish within ``BatchingConfig.timeout`` seconds of its submission
    (the reference's RequestTimeoutError, src/mlx_one/engine/actor.py:429-438)."""


# the token of a decode whose value is still on the device (chosen by a step that is in flight)
PENDING = -1


class Phase(enum.Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODE = "decode"
    FINISHED = "finished"


@dataclass
class Request:
    request_id: Any
    prompt: tuple[int, ...]
    options: TextGenerationOptions
    eos_token_ids: tuple[int, ...] = ()
    phase: Phase = Phase.WAITING
    fed: int = 0                                     # prompt tokens already run
    output: list[int] = field(default_factory=list)
    next_token: int | None = None                    # sampled, to be fed by the next step
    finish_reason: str | None = None     # "stop" | "length" | "cancelled" | "timeout" | "error"
    terminal_token_id: int | None = None
    cancelled: bool = False
    deadline: float | None = None                    # on the scheduler's clock; None: none
    error: BaseException | None = None               # why finish_reason is "error"
    pending: int = 0                                 # tokens drawn by steps whose result is not in yet

    @property
    def reserve_tokens(self) -> int:
        # the last sampled token is never fed back, so it needs no place in the cache
        return len(self.prompt) + self.options.max_tokens - 1


@dataclass
class Scheduled:
    """One request's share of a planned step."""

    request: Request
    tokens: tuple[int, ...]
    samples: bool                # logits at the last token are wanted and a token is drawn


class Scheduler:
    def __init__(self, config: BatchingConfig, cache: CacheManager, clock=time.monotonic) -> None:
        self.config = config
        self.cache = cache
        self.clock = clock
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self._decode_turn = 0
        self._single_turn = 0
        self._ids = itertools.count()

    # ------------------------------------------------------------------ requests

    def new_id(self) -> int:
        return next(self._ids)

    def submit(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if len(self.waiting) >= self.config.queue_size:
            raise QueueFullError(f"{len(self.waiting)} requests are already waiting")
        if not self.cache.fits_ever(request.reserve_tokens):
            raise CacheCapacityError(
                f"prompt of {len(request.prompt)} tokens plus {request.options.max_tokens} new "
                f"tokens can never fit into a cache of {self.cache.capacity_tokens} tokens",
                retryable=False)
        request.phase = Phase.WAITING
        if self.config.timeout and request.deadline is None:
            request.deadline = self.clock() + self.config.timeout
        self.waiting.append(request)

    def cancel(self, request: Request) -> None:
        """Takes effect between steps: the request is finished and freed by the next plan."""
        request.cancelled = True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ one step

    def _admit(self) -> None:
        for request in list(self.waiting):
            if len(self.running) >= self.config.max_sequences:
                break
            if request.cancelled:
                self.waiting.remove(request)
                self._finish(request, "cancelled", held=False)
                continue
            try:
                self.cache.open(request.request_id, reserve_tokens=request.reserve_tokens)
            except CacheCapacityError as error:
                if not error.retryable:
                    self.waiting.remove(request)
                    self._finish(request, "cancelled", held=False)
                continue                     # does not fit now; a younger one may
            self.waiting.remove(request)
            request.phase = Phase.PREFILL
            self.running.append(request)

    def plan(self) -> list[Scheduled]:
        """Frees cancelled requests and those whose time is up, admits waiting ones and chooses
        the next step."""
        now = self.clock()
        for request in [r for r in self.running if r.cancelled]:
            self._finish(request, "cancelled")
        for request in [r for r in self.running if r.deadline is not None and now >= r.deadline]:
            self._finish(request, "timeout")
        for request in [r for r in self.waiting if r.deadline is not None and now >= r.deadline]:
            self.waiting.remove(request)
            self._finish(request, "timeout", held=False)
        self._admit()
        config = self.config
        budget = config.max_scheduled_tokens
        step: list[Scheduled] = []
        # (a request whose last token is being drawn by a step in flight has nothing to run)
        decodes = [r for r in self.running if r.phase is Phase.DECODE
                   and len(r.output) + r.pending < r.options.max_tokens]
        prefills = [r for r in self.running if r.phase is Phase.PREFILL]
        if decodes and prefills:
            # decodes must not starve prompts: room is kept for a portion of the oldest one,
            # as the reference keeps room for the smallest waiting prefill
            # (src/mlx_one/engine/batching.py:89-95); with a budget of one they alternate
            oldest = prefills[0]
            room = min(len(oldest.prompt) - oldest.fed, config.prefill_chunk_size,
                       config.max_prefill_tokens, max(budget // 2, 1))
            if budget == 1:
                self._single_turn += 1
                room = self._single_turn % 2
            budget_for_decodes = max(budget - room, 0)
        else:
            budget_for_decodes = budget
        if len(decodes) > budget_for_decodes:
            start = self._decode_turn % len(decodes)
            decodes = (decodes[start:] + decodes[:start])[:budget_for_decodes]
            self._decode_turn += budget_for_decodes
        for request in decodes:
            token = PENDING if request.pending else request.next_token
            step.append(Scheduled(request, (token,), True))
        budget -= len(decodes)
        prefill_budget = min(budget, config.max_prefill_tokens)
        for request in self.running:
            if request.phase is not Phase.PREFILL or prefill_budget < 1:
                continue
            size = min(len(request.prompt) - request.fed, config.prefill_chunk_size,
                       prefill_budget)
            tokens = request.prompt[request.fed:request.fed + size]
            last = request.fed + size == len(request.prompt)
            step.append(Scheduled(request, tokens, last))
            prefill_budget -= size
        return step

    def advance(self, step: Sequence[Scheduled]) -> None:
        """Records that ``step`` has been launched: prompts move on by their portions, requests
        that draw a token in it count that token as pending. The next step can be planned from
        this before the step's tokens are known."""
        for item in step:
            request = item.request
            if request.phase is Phase.PREFILL:
                request.fed += len(item.tokens)
            if item.samples:
                request.phase = Phase.DECODE
                request.pending += 1

    def resolve(self, step: Sequence[Scheduled], sampled: Sequence[int],
                stop_at=None) -> list[Request]:
        """Records the tokens that an advanced step drew: ``sampled`` has one token per entry
        with ``samples``. Returns the requests that produced a token or finished. A request
        that has ended since the step was launched (cancelled, timed out, or ended by an earlier
        step's token that was read after this step's launch) drops its token.
        ``stop_at(request, token)`` is asked for every drawn token of a request that has stop
        strings: None lets the token in; a count means that the text with this token contains a
        stop string, and the request ends with reason "stop" holding only that many of its
        tokens (those before the match)."""
        touched, drawn = [], iter(sampled)
        for item in step:
            if not item.samples:
                continue
            token = int(next(drawn))
            request = item.request
            if request.phase is Phase.FINISHED:
                continue
            request.pending -= 1
            touched.append(request)
            if token in request.eos_token_ids and not request.options.ignore_eos:
                request.terminal_token_id = token
                self._finish(request, "stop")
                continue
            if stop_at is not None and request.options.stop:
                keep = stop_at(request, token)
                if keep is not None:
                    del request.output[keep:]
                    self._finish(request, "stop")
                    continue
            request.output.append(token)
            request.next_token = token
            if len(request.output) >= request.options.max_tokens:
                self._finish(request, "length")
        return touched

    def commit(self, step: Sequence[Scheduled], sampled: Sequence[int],
               stop_at=None) -> list[Request]:
        """``advance`` and ``resolve`` in one: a step whose tokens are known before the next
        step is planned."""
        self.advance(step)
        return self.resolve(step, sampled, stop_at)

    def fail(self, requests: Sequence[Request], error: BaseException) -> None:
        """Ends requests whose step could not be trusted (a kernel reported a fault, the step
        raised): their pages come back and whoever waits for them is given ``error``."""
        for request in requests:
            if request.phase is not Phase.FINISHED:
                request.error = error
                if request in self.waiting:
                    self.waiting.remove(request)
                    self._finish(request, "error", held=False)
                else:
                    self._finish(request, "error")

    def _finish(self, request: Request, reason: str, held: bool = True) -> None:
        request.finish_reason = reason
        request.phase = Phase.FINISHED
        request.next_token = None
        request.pending = 0
        if request in self.running:
            self.running.remove(request)
        if held and request.request_id in self.cache:
            self.cache.close(request.request_id)
