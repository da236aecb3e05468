"""The scheduler's decisions (host only): admission by reservation, portions under the token
budget, decode first, finishing and freeing, and what happens when pages run out."""

import pytest
import torch

from mlx_one_b200.cache import CacheCapacityError, CacheManager
from mlx_one_b200.engine.scheduler import (BatchingConfig, Phase, QueueFullError, Request,
                                           Scheduler)
from mlx_one_b200.parts.base import FixedState, PagedKeyValues
from mlx_one_b200.sampling import TextGenerationOptions

NEEDS = {0: FixedState((2, 8)), 1: PagedKeyValues(2, 16)}


def make(capacity=256, page=4, **config):
    cache = CacheManager(NEEDS, page_size=page, capacity_tokens=capacity, max_requests=8,
                         dtype=torch.float32, device="cpu", allocate=False)
    defaults = dict(max_sequences=4, queue_size=8, prefill_chunk_size=16,
                    max_scheduled_tokens=32, max_prefill_tokens=24)
    return Scheduler(BatchingConfig(**{**defaults, **config}), cache), cache


def request(scheduler, prompt_length, max_tokens=4, eos=(), **options):
    return Request(scheduler.new_id(), tuple(range(1, prompt_length + 1)),
                   TextGenerationOptions(max_tokens=max_tokens, **options), eos_token_ids=eos)


def run_step(scheduler, cache, token=100):
    """Plans a step, pretends to run it (grow + advance) and commits ``token`` for every draw."""
    step = scheduler.plan()
    for item in step:
        cache.grow(item.request.request_id, len(item.tokens))
        cache.advance(item.request.request_id, len(item.tokens))
    scheduler.commit(step, [token] * sum(1 for item in step if item.samples))
    cache.check()
    return step


def test_batching_config_has_the_reference_names_and_checks():
    config = BatchingConfig()
    assert (config.max_sequences, config.queue_size, config.prefill_chunk_size,
            config.max_scheduled_tokens, config.max_prefill_tokens) == (1, 8, 512, 2048, 1024)
    with pytest.raises(ValueError):
        BatchingConfig(prefill_chunk_size=0)
    assert config.timeout == 600.0
    with pytest.raises(ValueError):
        BatchingConfig(timeout=-1)


def test_prompts_are_cut_under_the_budget_and_decodes_come_first():
    scheduler, cache = make()
    a, b = request(scheduler, 40), request(scheduler, 10)
    scheduler.submit(a)
    scheduler.submit(b)
    step = run_step(scheduler, cache)
    # oldest first, 16 per request, 24 prompt tokens per step in all
    assert [(s.request, len(s.tokens), s.samples) for s in step] == [(a, 16, False), (b, 8, False)]
    step = run_step(scheduler, cache)
    assert [(s.request, len(s.tokens), s.samples) for s in step] == [(a, 16, False), (b, 2, True)]
    assert b.phase is Phase.DECODE and b.output == [100]
    step = run_step(scheduler, cache)
    assert [(s.request, s.tokens, s.samples) for s in step] == [(b, (100,), True),
                                                                (a, (33, 34, 35, 36, 37, 38, 39, 40), True)]
    assert a.phase is Phase.DECODE
    step = run_step(scheduler, cache)
    assert sorted(len(s.tokens) for s in step) == [1, 1]


def test_finish_by_length_and_by_end_token_frees_everything():
    scheduler, cache = make()
    by_length = request(scheduler, 3, max_tokens=2)
    by_eos = request(scheduler, 3, max_tokens=9, eos=(100,))
    ignoring = request(scheduler, 3, max_tokens=2, eos=(100,), ignore_eos=True)
    for r in (by_length, by_eos, ignoring):
        scheduler.submit(r)
    run_step(scheduler, cache)
    assert by_eos.finish_reason == "stop" and by_eos.output == [] and by_eos.terminal_token_id == 100
    run_step(scheduler, cache)
    assert by_length.finish_reason == "length" and by_length.output == [100, 100]
    assert ignoring.finish_reason == "length" and ignoring.output == [100, 100]
    assert not scheduler.has_work() and not cache.requests()
    assert cache.stats().pages_free == cache.stats().pages_total


def test_when_pages_run_out_requests_wait_and_nothing_is_preempted():
    """16 pages of 4 tokens. Each request reserves its whole future (prompt + max_tokens - 1):
    the third does not fit beside the first two and waits until one ends; a younger request
    that does fit is admitted past it."""
    scheduler, cache = make(capacity=64, max_sequences=8)
    first, second = request(scheduler, 20, max_tokens=5), request(scheduler, 20, max_tokens=5)
    third = request(scheduler, 20, max_tokens=5)
    small = request(scheduler, 3, max_tokens=2)
    for r in (first, second, third, small):
        scheduler.submit(r)
    run_step(scheduler, cache)
    assert [r.phase for r in (first, second, third, small)] == [
        Phase.PREFILL, Phase.PREFILL, Phase.WAITING, Phase.PREFILL]    # small got past third
    assert small.request_id in cache and third.request_id not in cache
    for _ in range(50):
        if third.phase is not Phase.WAITING:
            break
        run_step(scheduler, cache)
        assert first.phase is not Phase.WAITING and second.phase is not Phase.WAITING
    assert third.phase is not Phase.WAITING
    assert first.phase is Phase.FINISHED or second.phase is Phase.FINISHED
    for _ in range(50):
        if scheduler.has_work():
            run_step(scheduler, cache)
    assert all(r.finish_reason == "length" for r in (first, second, third, small))
    assert third.output == [100] * 5


def test_a_request_that_can_never_fit_is_refused_at_once():
    scheduler, cache = make(capacity=32)
    with pytest.raises(CacheCapacityError) as caught:
        scheduler.submit(request(scheduler, 30, max_tokens=8))
    assert not caught.value.retryable
    scheduler.submit(request(scheduler, 30, max_tokens=3))
    with pytest.raises(ValueError):
        scheduler.submit(Request(99, (), TextGenerationOptions()))


def test_queue_limit_and_cancel():
    scheduler, cache = make(max_sequences=1, queue_size=2)
    running = request(scheduler, 5, max_tokens=50)
    scheduler.submit(running)
    run_step(scheduler, cache)
    waiting = [request(scheduler, 5), request(scheduler, 5)]
    for r in waiting:
        scheduler.submit(r)
    with pytest.raises(QueueFullError):
        scheduler.submit(request(scheduler, 5))
    scheduler.cancel(running)
    scheduler.cancel(waiting[0])
    step = run_step(scheduler, cache)
    assert running.finish_reason == "cancelled" and waiting[0].finish_reason == "cancelled"
    assert [s.request for s in step] == [waiting[1]]
    assert running.request_id not in cache


def test_more_decodes_than_budget_take_turns():
    scheduler, cache = make(max_sequences=6, max_scheduled_tokens=4, prefill_chunk_size=4,
                            max_prefill_tokens=4)
    requests = [request(scheduler, 2, max_tokens=20) for _ in range(6)]
    for r in requests:
        scheduler.submit(r)
    for _ in range(40):
        if all(r.phase is Phase.DECODE for r in requests):
            break
        run_step(scheduler, cache)
    assert all(r.phase is Phase.DECODE for r in requests)     # decodes did not starve prompts
    counts = {r.request_id: len(r.output) for r in requests}
    for _ in range(6):
        assert len(run_step(scheduler, cache)) == 4
    gained = [len(r.output) - counts[r.request_id] for r in requests]
    assert gained == [4] * 6


def test_budget_of_one_alternates_between_decode_and_prompt():
    scheduler, cache = make(max_sequences=2, max_scheduled_tokens=1, prefill_chunk_size=1,
                            max_prefill_tokens=1)
    a, b = request(scheduler, 1, max_tokens=30), request(scheduler, 4, max_tokens=2)
    scheduler.submit(a)
    run_step(scheduler, cache)
    scheduler.submit(b)
    kinds = []
    for _ in range(8):
        step = run_step(scheduler, cache)
        assert len(step) == 1
        kinds.append(step[0].request is a)
    assert True in kinds and False in kinds and b.phase is Phase.DECODE


def test_a_request_whose_time_is_up_ends_and_frees_its_pages():
    """``timeout`` seconds after its submission a request ends with the reason "timeout",
    whether it runs or still waits; its pages and slot come back; others go on. 0: never."""
    scheduler, cache = make(max_sequences=1, timeout=10.0)
    now = [100.0]
    scheduler.clock = lambda: now[0]
    running = request(scheduler, 5, max_tokens=50)
    scheduler.submit(running)
    run_step(scheduler, cache)
    waiting = request(scheduler, 5, max_tokens=50)
    now[0] = 105.0
    scheduler.submit(waiting)
    assert (running.deadline, waiting.deadline) == (110.0, 115.0)
    run_step(scheduler, cache)
    assert running.phase is Phase.DECODE and waiting.phase is Phase.WAITING
    now[0] = 110.0
    step = run_step(scheduler, cache)
    assert running.finish_reason == "timeout" and running.request_id not in cache
    assert [s.request for s in step] == [waiting]            # the slot went to the next one
    now[0] = 200.0
    late = request(scheduler, 5)
    scheduler.submit(late)
    now[0] = 215.0
    run_step(scheduler, cache)
    assert waiting.finish_reason == "timeout" and late.finish_reason == "timeout"
    assert not scheduler.has_work()
    stats = cache.stats()
    assert stats.pages_free == stats.pages_total and stats.slots_free == stats.slots_total
    never, cache = make(timeout=0)
    patient = request(never, 5)
    never.submit(patient)
    assert patient.deadline is None


def test_a_step_can_be_planned_before_the_last_one_is_resolved():
    """``advance`` tells the scheduler that a step was launched; the next plan then holds
    decodes whose token is still pending, and prompt portions that follow on. ``resolve`` brings
    the tokens later: a request that an earlier token has ended drops the token that a later
    step drew for it, and a request that is drawing its last token is not planned again."""
    from mlx_one_b200.engine.scheduler import PENDING

    scheduler, cache = make(max_scheduled_tokens=32, max_prefill_tokens=24, prefill_chunk_size=16)
    a = request(scheduler, 3, max_tokens=3, eos=(7,))
    b = request(scheduler, 20, max_tokens=2)
    scheduler.submit(a)
    scheduler.submit(b)

    def launch():
        step = scheduler.plan()
        for item in step:
            cache.grow(item.request.request_id, len(item.tokens))
            cache.advance(item.request.request_id, len(item.tokens))
        scheduler.advance(step)
        return step

    first = launch()                                  # a's whole prompt (draws), 16 tokens of b
    assert [(s.request, len(s.tokens), s.samples) for s in first] == [(a, 3, True), (b, 16, False)]
    assert a.pending == 1 and a.phase is Phase.DECODE and b.fed == 16
    second = launch()                                 # planned before a's first token is known
    assert [(s.request, s.tokens, s.samples) for s in second] == \
        [(a, (PENDING,), True), (b, tuple(range(17, 21)), True)]
    assert a.pending == 2 and b.pending == 1
    assert scheduler.resolve(first, [5]) == [a] and a.output == [5] and a.pending == 1
    third = launch()                                  # a draws its third (last) token; b decodes
    assert [(s.request, s.tokens) for s in third] == [(a, (PENDING,)), (b, (PENDING,))]
    assert scheduler.plan() == []                     # both are drawing their last tokens
    # the second step's token for a is the end-of-sequence token: a ends, b goes on
    touched = scheduler.resolve(second, [7, 9])
    assert touched == [a, b] and a.phase is Phase.FINISHED and a.finish_reason == "stop"
    assert a.output == [5] and a.terminal_token_id == 7 and b.output == [9]
    assert a.request_id not in cache                  # its pages are back
    # the third step's token for a is dropped; b's second token ends it by length
    touched = scheduler.resolve(third, [11, 12])
    assert touched == [b] and a.output == [5] and b.output == [9, 12]
    assert b.finish_reason == "length" and not scheduler.has_work()
    cache.check()
    assert not cache.requests()
