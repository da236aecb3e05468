"""The cache manager: pages for keys and values, slots for fixed-size state.

Cache entries (one per layer call that keeps something) with equal needs form a group.
A paged group owns one pool of pages; a request has one block table per paged group and
all entries of the group use the same page numbers, each in its own storage. Groups with
a window give a page back as soon as every position in it has left the window of the next
query. A fixed-state group owns a pool of slots; a request has one slot per group.

Storage (on the device, in place):
  paged group   [entries, 2, pages, kv_heads, page_size, head_dim]
  state group   [entries, slots, *shape]

Requests are opened, grown before a step (``grow``), advanced after it (``advance``) and
closed. A request may reserve its whole future when it is opened; growth then draws on
the reservation and cannot fail. Unreserved requests take pages that no reservation
claims. The reference reserves at admission in the same way
(src/mlx_one/engine/cache_manager.py:217-341) and gives everything back on release
(:686-714).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

import torch

from ..parts.base import FixedState, PagedKeyValues, PagedView, StateView
from .errors import CacheCapacityError, CacheOwnershipError
from .pools import IndexPool


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class PagedGroup:
    need: PagedKeyValues
    entries: tuple[int, ...]
    pool: IndexPool
    storage: torch.Tensor | None
    promised: int = 0                     # reserved by requests but not yet taken


@dataclass
class StateGroup:
    need: FixedState
    entries: tuple[int, ...]
    pool: IndexPool
    storage: torch.Tensor | None


@dataclass
class RequestCache:
    """What one request holds."""

    request_id: Any
    index: int = 0                                          # a number of its own among live requests
    length: int = 0                                         # tokens committed
    tables: list[list[int]] = field(default_factory=list)   # per paged group; -1 = given back
    live: list[int] = field(default_factory=list)           # pages held, per paged group
    promised: list[int] = field(default_factory=list)       # reservation left, per paged group
    slots: list[int] = field(default_factory=list)          # per state group
    reserved_tokens: int | None = None


@dataclass(frozen=True)
class CacheStats:
    pages_total: tuple[int, ...]
    pages_free: tuple[int, ...]
    pages_promised: tuple[int, ...]
    pages_low_water: tuple[int, ...]
    slots_total: tuple[int, ...]
    slots_free: tuple[int, ...]
    requests: int


class CacheManager:
    def __init__(self, needs: Mapping[int, Any], *, page_size: int, capacity_tokens: int,
                 max_requests: int, dtype: torch.dtype, device, max_step_tokens: int = 1 << 30,
                 allocate: bool = True) -> None:
        """``needs``: cache entry -> ``PagedKeyValues`` | ``FixedState``.
        ``capacity_tokens``: tokens that all live requests may hold together; every paged
        group gets ceil(capacity_tokens / page_size) pages."""
        if page_size < 1 or capacity_tokens < 1 or max_requests < 1:
            raise ValueError("page_size, capacity_tokens and max_requests must be positive")
        self.page_size = page_size
        self.capacity_tokens = capacity_tokens
        self.max_requests = max_requests
        self.max_step_tokens = max_step_tokens
        self.dtype = dtype
        self.device = torch.device(device)
        pages = ceil_div(capacity_tokens, page_size)
        by_need: dict[Any, list[int]] = {}
        for entry in sorted(needs):
            by_need.setdefault(needs[entry], []).append(entry)
        self.paged: list[PagedGroup] = []
        self.states: list[StateGroup] = []
        self._where: dict[int, tuple[str, int, int]] = {}
        for need, entries in by_need.items():
            if isinstance(need, PagedKeyValues):
                storage = None
                if allocate:
                    # one page beyond the pool's: the scratch page (see ``scratch_page``)
                    storage = torch.zeros((len(entries), 2, pages + 1, need.kv_heads, page_size,
                                           need.head_dim), dtype=dtype, device=self.device)
                group = len(self.paged)
                self.paged.append(PagedGroup(need, tuple(entries), IndexPool(pages, "page"),
                                             storage))
                for i, entry in enumerate(entries):
                    self._where[entry] = ("paged", group, i)
            elif isinstance(need, FixedState):
                storage = None
                if allocate:
                    kind = torch.float32 if need.dtype == "float32" else dtype
                    # one slot beyond the pool's: the scratch slot
                    storage = torch.zeros((len(entries), max_requests + 1, *need.shape),
                                          dtype=kind, device=self.device)
                group = len(self.states)
                self.states.append(StateGroup(need, tuple(entries),
                                              IndexPool(max_requests, "slot"), storage))
                for i, entry in enumerate(entries):
                    self._where[entry] = ("state", group, i)
            else:
                raise TypeError(f"cache entry {entries[0]} has an unknown need {need!r}")
        self._requests: dict[Any, RequestCache] = {}
        self._indices = IndexPool(max_requests, "request number")
        # A page and a slot that no request ever gets, in every group. The step function points
        # the filler entries there with which it rounds a step's shape up (so that steps of few
        # distinct shapes can be replayed as CUDA graphs): what fillers write lands there and
        # is never read by a request.
        self.scratch_page = pages
        self.scratch_slot = max_requests

    # ------------------------------------------------------------------ sizes

    def pages_for(self, group: PagedGroup, tokens: int) -> int:
        """Most pages a request of ``tokens`` tokens holds in ``group`` at any time."""
        whole = ceil_div(tokens, self.page_size)
        if group.need.window is None:
            return whole
        # keys of the last window-1 positions, the step's own tokens, and one ragged edge
        step = min(self.max_step_tokens, tokens)
        return min(whole, ceil_div(group.need.window - 1 + step, self.page_size) + 1)

    def fits_ever(self, tokens: int) -> bool:
        return all(self.pages_for(g, tokens) <= g.pool.count for g in self.paged)

    def fits_now(self, tokens: int) -> bool:
        if any(g.pool.free < 1 for g in self.states):
            return False
        return all(self.pages_for(g, tokens) <= g.pool.free - g.promised for g in self.paged)

    # ------------------------------------------------------------------ lifecycle

    def open(self, request_id: Any, reserve_tokens: int | None = None) -> RequestCache:
        """Registers a request, gives it a zeroed slot in every state group and, if
        ``reserve_tokens`` is given, sets pages aside for that many tokens."""
        if request_id in self._requests:
            raise CacheOwnershipError(f"request {request_id!r} is already open")
        if len(self._requests) >= self.max_requests:
            raise CacheCapacityError("no request slot free", retryable=True)
        if reserve_tokens is not None:
            if not self.fits_ever(reserve_tokens):
                raise CacheCapacityError(
                    f"{reserve_tokens} tokens can never fit into {self.capacity_tokens}",
                    retryable=False)
            if not self.fits_now(reserve_tokens):
                raise CacheCapacityError(f"{reserve_tokens} tokens do not fit now",
                                         retryable=True)
        cache = RequestCache(request_id, index=self._indices.take(),
                             reserved_tokens=reserve_tokens)
        for group in self.paged:
            cache.tables.append([])
            cache.live.append(0)
            want = 0 if reserve_tokens is None else self.pages_for(group, reserve_tokens)
            cache.promised.append(want)
            group.promised += want
        for group in self.states:
            slot = group.pool.take()
            cache.slots.append(slot)
            if group.storage is not None:
                group.storage[:, slot].zero_()
        self._requests[request_id] = cache
        return cache

    def get(self, request_id: Any) -> RequestCache:
        try:
            return self._requests[request_id]
        except KeyError:
            raise CacheOwnershipError(f"request {request_id!r} is not open") from None

    def __contains__(self, request_id: Any) -> bool:
        return request_id in self._requests

    def grow(self, request_id: Any, new_tokens: int) -> None:
        """Makes sure every position below length + new_tokens has a page. Takes nothing
        if any group cannot serve the whole growth."""
        cache = self.get(request_id)
        target = cache.length + new_tokens
        if cache.reserved_tokens is not None and target > cache.reserved_tokens:
            raise CacheCapacityError(
                f"request {request_id!r} grows to {target} tokens beyond its reservation "
                f"of {cache.reserved_tokens}", retryable=False)
        wanted = []
        for index, group in enumerate(self.paged):
            more = max(ceil_div(target, self.page_size) - len(cache.tables[index]), 0)
            from_promise = min(more, cache.promised[index])
            open_pages = group.pool.free - group.promised
            if more - from_promise > open_pages:
                raise CacheCapacityError(
                    f"request {request_id!r} needs {more} more pages, {open_pages} are free",
                    retryable=True)
            wanted.append((more, from_promise))
        for index, (more, from_promise) in enumerate(wanted):
            group = self.paged[index]
            for _ in range(more):
                cache.tables[index].append(group.pool.take())
            cache.live[index] += more
            cache.promised[index] -= from_promise
            group.promised -= from_promise

    def advance(self, request_id: Any, new_tokens: int) -> None:
        """Commits ``new_tokens`` tokens and gives back pages that a window has passed."""
        cache = self.get(request_id)
        cache.length += new_tokens
        for index, group in enumerate(self.paged):
            window = group.need.window
            if window is None:
                continue
            # the next query sits at position >= length and reads keys > query - window
            first_needed = cache.length - window + 1
            table = cache.tables[index]
            for block in range(min(max(first_needed, 0) // self.page_size, len(table))):
                if table[block] >= 0:
                    group.pool.give_back(table[block])
                    table[block] = -1
                    cache.live[index] -= 1
                    if cache.reserved_tokens is not None:
                        cache.promised[index] += 1
                        group.promised += 1

    def close(self, request_id: Any) -> None:
        """Gives back everything the request holds or has reserved."""
        cache = self._requests.pop(request_id, None)
        if cache is None:
            raise CacheOwnershipError(f"request {request_id!r} is not open")
        for index, group in enumerate(self.paged):
            for page in reversed(cache.tables[index]):
                if page >= 0:
                    group.pool.give_back(page)
            group.promised -= cache.promised[index]
        for index, group in enumerate(self.states):
            group.pool.give_back(cache.slots[index])
        self._indices.give_back(cache.index)

    def close_all(self) -> None:
        for request_id in list(self._requests):
            self.close(request_id)

    # ------------------------------------------------------------------ views and stats

    def locate(self, entry: int) -> tuple[str, int, int]:
        """(kind, group, index in the group) of a cache entry."""
        return self._where[entry]

    def view(self, entry: int, tables: list[torch.Tensor], slots: list[torch.Tensor]):
        """The view of one cache entry for a step, given the step's device block tables
        (one per paged group) and slot lists (one per state group)."""
        kind, group, index = self._where[entry]
        if kind == "paged":
            g = self.paged[group]
            return PagedView(g.storage[index], tables[group], self.page_size, g.need)
        g = self.states[group]
        return StateView(g.storage[index], slots[group], g.need)

    def requests(self) -> tuple[Any, ...]:
        return tuple(self._requests)

    def stats(self) -> CacheStats:
        return CacheStats(
            pages_total=tuple(g.pool.count for g in self.paged),
            pages_free=tuple(g.pool.free for g in self.paged),
            pages_promised=tuple(g.promised for g in self.paged),
            pages_low_water=tuple(g.pool.low_water for g in self.paged),
            slots_total=tuple(g.pool.count for g in self.states),
            slots_free=tuple(g.pool.free for g in self.states),
            requests=len(self._requests))

    def check(self) -> None:
        """Every page and slot is either free or held by exactly one request."""
        for index, group in enumerate(self.paged):
            seen: set[int] = set()
            for cache in self._requests.values():
                pages = [p for p in cache.tables[index] if p >= 0]
                if len(pages) != cache.live[index]:
                    raise CacheOwnershipError("live page count is out of step")
                for page in pages:
                    if page in seen:
                        raise CacheOwnershipError(f"page {page} is held twice")
                    seen.add(page)
            if seen != group.pool.held():
                raise CacheOwnershipError("held pages and block tables disagree: a page is lost")
            if group.promised != sum(c.promised[index] for c in self._requests.values()):
                raise CacheOwnershipError("promised pages are out of step")
            if group.promised > group.pool.free:
                raise CacheOwnershipError("more pages are promised than free")
        for index, group in enumerate(self.states):
            slots = [c.slots[index] for c in self._requests.values()]
            if len(set(slots)) != len(slots) or set(slots) != group.pool.held():
                raise CacheOwnershipError("slots and requests disagree")
