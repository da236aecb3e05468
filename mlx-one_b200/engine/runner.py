"""The step function: one ragged batch of (request, its next tokens) through the model.

A step takes, for every request in it, the tokens that come next (a portion of a prompt, or
one decoded token), runs exactly these tokens as one batch against what earlier steps left
in the cache, appends their keys, values and state, and returns the 32-bit logits at the
places asked for. A decoded token is simply a portion of length one, so prompts and decodes
mix freely. The reference runs one phase per batch and pads to the widest row
(src/mlx_one/engine/hybrid.py:115-252); here nothing is padded.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..parts.base import NoHostValues, StepContext
from ..parts.model import Model


@dataclass
class StepEntry:
    """One request's share of a step. ``want``: places among ``tokens`` whose logits are
    returned (in this order)."""

    request_id: Any
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)
    # the (single) token is the one that an earlier greedy step chose for this request and
    # published on the device; ``tokens`` then only gives the count
    from_device: bool = False


def _align(value: int, to: int = 4) -> int:
    return -(-value // to) * to


@dataclass
class _DecodeGraph:
    """A captured decode-only step: its own metadata buffer (so that addresses never
    change), the graph, and the tensors it leaves its results in."""

    meta: torch.Tensor
    graph: Any = None
    logits: torch.Tensor | None = None
    uses: int = 0
    counter: torch.Tensor | None = None
    record: torch.Tensor | None = None
    _record: torch.Tensor | None = None

    def record_buffer(self, like: torch.Tensor) -> torch.Tensor:
        """A buffer at a fixed address that holds at least as many steps as ``like``."""
        if self._record is None:
            self._record = torch.zeros((max(like.shape[0], 4096), like.shape[1]),
                                       dtype=torch.int32, device=like.device)
        if like.shape[0] > self._record.shape[0]:
            raise ValueError(f"at most {self._record.shape[0]} steps in one decode loop")
        return self._record


class Runner:
    def __init__(self, model: Model, cache: CacheManager) -> None:
        self.model = model
        self.cache = cache
        self.ops = model.ops
        self.device = model.runtime.device
        self._staging: list[torch.Tensor | None] = [None, None]
        self._events: list[Any] = [None, None]
        self._device_buffer: torch.Tensor | None = None
        self._turn = 0
        self.steps = 0
        self.last_shape = (0, 0)
        self.last_meta_bytes = 0
        self.last_greedy: torch.Tensor | None = None
        # what the host reads back after a step that chose tokens: int32, the tokens of the
        # wanted rows (``last_greedy``, then any filler rows'), then the kernels' error flag
        self.last_report: torch.Tensor | None = None
        # an event that the next step's kernels (not its metadata copy) wait for: the caller's
        # copy of ``last_report`` to the host on a stream of its own
        self.wait_before_kernels: Any = None
        # tokens chosen on the device, by request number (see StepEntry.from_device)
        # (one entry more than there are requests: where filler rows publish theirs)
        self.published = torch.zeros(cache.max_requests + 1, dtype=torch.int32,
                                     device=self.device)
        # CUDA graphs of steps, keyed by shape (requests, tokens, table widths, wanted rows, ...)
        # (only models whose parts all say that they can be captured: see Part.capturable)
        self.use_graphs = self.device.type == "cuda" and model.capturable
        self._graphs: dict[tuple, _DecodeGraph] = {}
        self.graph_replays = 0
        self.graph_captures = 0
        self.graph_memory_bytes = 0         # device memory that captures have added to the allocator
        # steps with portions: captured at their third occurrence if they have at most this many
        # tokens (larger ones keep the GPU busy longer than the host needs to launch them)
        self.graph_token_limit = 1024
        self.portion_graphs = 64
        self._portion_keys: list[tuple] = []
        # Steps that may be captured have their shape rounded up with filler entries, so that
        # the steps of a changing batch fall on few shapes: tokens to a multiple of
        # ``token_bucket`` (16 up to 128 tokens), requests and wanted rows to a multiple of
        # ``request_bucket`` (decode-only steps of up to that many requests stay as they are)
        self.token_bucket = 64
        self.request_bucket = 8
        # decode-only shapes kept; the least recently used ones are dropped beyond this. (Every
        # graph keeps a memory pool of its own: its logits stay valid until its next replay,
        # whatever other graphs run in between.)
        self.decode_graphs = 48
        self._decode_keys: list[tuple] = []
        if self.use_graphs:
            # library handles must exist before a capture begins
            warm = torch.zeros((8, 8), dtype=torch.bfloat16, device=self.device)
            torch.mm(warm, warm)

    # ------------------------------------------------------------------ staging

    def _host_buffer(self, size: int) -> torch.Tensor:
        """A host int32 buffer of at least ``size`` entries whose last copy has landed."""
        self._turn ^= 1
        turn = self._turn
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        buffer = self._staging[turn]
        if buffer is None or buffer.numel() < size:
            capacity = max(1024, 1 << (size - 1).bit_length())
            buffer = torch.empty(capacity, dtype=torch.int32,
                                 pin_memory=self.device.type == "cuda")
            self._staging[turn] = buffer
        if self._device_buffer is None or self._device_buffer.numel() < buffer.numel():
            self._device_buffer = torch.empty(buffer.numel(), dtype=torch.int32,
                                              device=self.device)
        return buffer

    # ------------------------------------------------------------------ the step

    def step(self, entries: Sequence[StepEntry], greedy: bool = False,
             draw: Sequence[tuple] | None = None) -> torch.Tensor | None:
        """See ``_step``. With ``greedy`` the argmax of every wanted row, with ``draw`` a sampled
        token, is computed in the same launch sequence (inside the CUDA graph of a captured
        step), published for steps that take their input from the device, and left in
        ``last_greedy`` as int32 [wanted] on the device. ``draw`` gives for every wanted row
        (temperature, top_k, top_p, seed, tokens drawn so far); a temperature of 0 is greedy."""
        return self._step(entries, greedy=greedy, draw=draw)

    def decode_steps(self, entries: Sequence[StepEntry], steps: int,
                     events: tuple | None = None) -> torch.Tensor:
        """``steps`` greedy decode steps in a row without the host in between: every entry
        brings its next token; each step's argmax becomes the next step's input on the
        device. Pages for all steps are taken first. Returns the chosen tokens as int32
        [steps, requests] on the device (not synchronised). ``events``: two CUDA events that
        are recorded directly before the first step's launch and after the last one's, for
        timing the steps without the host's preparation of the loop."""
        if steps < 1 or any(len(e.tokens) != 1 for e in entries):
            raise ValueError("decode_steps takes one token per request and at least one step")
        limit = self.model.spec.max_positions
        for entry in entries:
            if self.cache.get(entry.request_id).length + steps > limit:
                raise ValueError(f"request {entry.request_id!r} would pass the model's "
                                 f"{limit} positions")
        for entry in entries:
            self.cache.grow(entry.request_id, steps)
        entries = [StepEntry(e.request_id, e.tokens, (0,)) for e in entries]
        record = torch.zeros((steps, len(entries)), dtype=torch.int32, device=self.device)
        return self._step(entries, loop=(steps, record, events))

    def _step(self, entries: Sequence[StepEntry], loop=None, greedy: bool = False, draw=None):
        """Runs the entries as one batch. Returns float32 logits [wanted, vocab] on the
        device in the order of the entries and of their ``want``, or None if nothing is
        wanted. Raises before touching any state if the batch is malformed or pages run
        out (``CacheCapacityError``)."""
        if not entries:
            return None
        vocab = self.model.spec.vocab_size
        seen = set()
        arrays: list[np.ndarray] = []
        for entry in entries:
            if entry.request_id in seen:
                raise ValueError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            if len(entry.tokens) < 1:
                raise ValueError(f"request {entry.request_id!r} brings no tokens")
            ids = np.asarray(entry.tokens, dtype=np.int64)
            if entry.from_device:
                if len(ids) != 1:
                    raise ValueError("a token taken from the device is a single token")
                ids = np.zeros(1, dtype=np.int64)
            if ids.ndim != 1 or ids.min() < 0 or ids.max() >= vocab:
                raise ValueError(f"request {entry.request_id!r} has a token outside the "
                                 f"vocabulary of {vocab}")
            arrays.append(ids)
            for place in entry.want:
                if not 0 <= int(place) < len(entry.tokens):
                    raise ValueError(f"wanted place {place} is outside the request's tokens")
            limit = self.model.spec.max_positions
            held = self.cache.get(entry.request_id).length
            if held + len(entry.tokens) > limit:
                raise ValueError(f"request {entry.request_id!r} would pass the model's "
                                 f"{limit} positions")
        if loop is None:
            for entry in entries:
                self.cache.grow(entry.request_id, len(entry.tokens))

        requests = len(entries)
        tokens = sum(len(e.tokens) for e in entries)
        wanted = sum(len(e.want) for e in entries)
        # the requests at the head of the step that bring a single token each (running decodes,
        # as the scheduler orders a step): kernels may treat them apart from the portions
        singles = next((i for i, e in enumerate(entries) if len(e.tokens) != 1), requests)
        caches = [self.cache.get(e.request_id) for e in entries]
        paged, states = self.cache.paged, self.cache.states
        widths = [_align(max(max(len(c.tables[g]) for c in caches), 1), 8)
                  for g in range(len(paged))]
        decode_only = (self.use_graphs or loop is not None) and tokens == requests
        # Steps with portions are captured too when their shape comes back and they are small
        # enough to be bound by the host's launches rather than by the GPU's work.
        portions = (self.use_graphs and not decode_only and loop is None
                    and tokens <= self.graph_token_limit)
        fill_singles = fill_others = fill_tokens = fill_wanted = 0
        if decode_only or portions:
            # few distinct widths, so that few graphs are captured
            widths = [max(1 << (w - 1).bit_length(), 32) for w in widths]
        if self.use_graphs and loop is None and (decode_only or portions):
            fill_singles, fill_others, fill_tokens, fill_wanted = self._fill(
                singles, requests - singles, tokens - singles, wanted)
        real_wanted = wanted
        # the step as it is packed: real singles, filler singles, the other entries, other fillers
        # (a filler is a request without history whose pages and slot are the scratch ones)
        packed: list[tuple] = [(e, c, a) for e, c, a in
                               zip(entries[:singles], caches[:singles], arrays[:singles])]
        packed += [(None, None, 1)] * fill_singles
        packed += [(e, c, a) for e, c, a in
                   zip(entries[singles:], caches[singles:], arrays[singles:])]
        for filler in range(fill_others):
            packed.append((None, None, fill_tokens - (fill_others - 1) if filler == 0 else 1))
        singles += fill_singles
        requests += fill_singles + fill_others
        tokens += fill_singles + fill_tokens
        wanted += fill_wanted

        # one packed int32 buffer: five per-token and per-request lists, block tables, slots
        offsets, cursor = {}, 0
        def region(name: str, size: int) -> None:
            nonlocal cursor
            offsets[name] = (cursor, size)
            cursor = _align(cursor + size)
        region("token_ids", tokens)
        region("positions", tokens)
        region("token_request", tokens)
        region("request_start", requests + 1)
        region("history", requests)
        region("rows", max(wanted, 1))
        region("token_source", tokens)            # published token to take, or -1
        region("want_index", max(wanted, 1))       # request number of each wanted row
        for g in range(len(paged)):
            region(f"table{g}", requests * widths[g])
        for g in range(len(states)):
            region(f"slots{g}", requests)
        if draw is not None:
            if len(draw) != real_wanted or not real_wanted:
                raise ValueError("draw needs one entry per wanted row")
            # the sampling kernel's arguments, per wanted row: floats by their bits, the seed
            # as two 32-bit halves
            for name in ("draw_temperature", "draw_top_k", "draw_top_p", "draw_step"):
                region(name, wanted)
            region("draw_seed", 2 * wanted)
            self.ops.reserve_sample_scratch(self.cache.max_requests + self.request_bucket, vocab)
        host = self._host_buffer(cursor)
        data = host.numpy()
        self.last_meta_bytes = 4 * cursor

        def put(name: str, values) -> None:
            start, size = offsets[name]
            data[start:start + size] = values

        starts, history, rows, want_index = [0], [], [], []
        source_at = offsets["token_source"][0]
        data[source_at:source_at + tokens] = -1
        ids_at = offsets["token_ids"][0]
        positions_at = offsets["positions"][0]
        request_at = offsets["token_request"][0]
        tables = []
        for g in range(len(paged)):
            start, size = offsets[f"table{g}"]
            tables.append(data[start:start + size].reshape(requests, widths[g]))
        slot_lists: list[list[int]] = [[] for _ in states]
        for r, (entry, cache, ids) in enumerate(packed):
            first = starts[-1]
            if entry is None:                       # a filler with ``ids`` tokens
                n, length = ids, 0
                data[ids_at + first:ids_at + first + n] = 0
                for g, table in enumerate(tables):
                    table[r] = self.cache.scratch_page
                for slots in slot_lists:
                    slots.append(self.cache.scratch_slot)
            else:
                n, length = len(ids), cache.length
                data[ids_at + first:ids_at + first + n] = ids
                rows.extend(first + int(place) for place in entry.want)
                want_index.extend([cache.index] * len(entry.want))
                if entry.from_device:
                    data[source_at + first] = cache.index
                for g, table in enumerate(tables):
                    held = cache.tables[g]
                    table[r, :len(held)] = held
                    table[r, len(held):] = -1
                for g, slots in enumerate(slot_lists):
                    slots.append(cache.slots[g])
            data[positions_at + first:positions_at + first + n] = np.arange(
                length, length + n, dtype=np.int32)
            data[request_at + first:request_at + first + n] = r
            starts.append(first + n)
            history.append(length)
        # filler rows of logits: any valid token row; their tokens are published to the spare entry
        rows.extend([0] * fill_wanted)
        # every token's row wanted, in order: the logits need no picking of rows
        every_row = wanted == tokens and rows == list(range(tokens))
        want_index.extend([self.cache.max_requests] * fill_wanted)
        if draw is not None:
            draw = list(draw) + [(1.0, 0, 1.0, 0, 0)] * fill_wanted
            def view(name, kind):
                start, size = offsets[name]
                return data[start:start + size].view(kind)
            view("draw_temperature", np.float32)[:] = [d[0] for d in draw]
            view("draw_top_k", np.int32)[:] = [d[1] or 0 for d in draw]
            view("draw_top_p", np.float32)[:] = [d[2] for d in draw]
            view("draw_seed", np.int64)[:] = [d[3] for d in draw]
            view("draw_step", np.int32)[:] = [d[4] for d in draw]
        put("want_index", want_index if want_index else [0])
        put("request_start", starts)
        put("history", history)
        put("rows", rows if rows else [0])
        for g, slots in enumerate(slot_lists):
            put(f"slots{g}", slots)

        device = self._device_buffer
        captured = None
        if decode_only or portions:
            key = (requests, singles, tokens, tuple(widths), wanted, loop is not None, greedy,
                   draw is not None, any(e.from_device for e in entries), every_row)
            captured = self._graphs.get(key)
            if captured is None:
                captured = _DecodeGraph(torch.empty(cursor, dtype=torch.int32,
                                                    device=self.device))
                self._graphs[key] = captured
            if portions:
                self._forget_old_portion_graphs(key)
            elif loop is None:
                self._forget_old_decode_graphs(key)
            device = captured.meta
        device[:cursor].copy_(host[:cursor], non_blocking=True)
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
            self._events[self._turn] = event
            if self.wait_before_kernels is not None:
                # (a copy on another stream that reads what this step's kernels will overwrite:
                # it has had this step's metadata copy to finish in, so the wait costs nothing)
                torch.cuda.current_stream(self.device).wait_event(self.wait_before_kernels)
                self.wait_before_kernels = None

        def on_device(name: str) -> torch.Tensor:
            start, size = offsets[name]
            return device[start:start + size]

        tables = [on_device(f"table{g}").view(requests, widths[g]) for g in range(len(paged))]
        slots = [on_device(f"slots{g}") for g in range(len(states))]
        views = {entry: self.cache.view(entry, tables, slots) for entry in self.model.cache_needs}
        if captured is None or not self.use_graphs:
            max_portion = max(len(e.tokens) for e in entries)
            max_context = max(c.length + len(e.tokens) for c, e in zip(caches, entries))
            host = {"history": history, "request_start": starts}
        else:
            # bounds that hold for every step of this shape, however its tokens are split
            max_portion = tokens - requests + 1
            max_context = min([self.model.spec.max_positions] +
                              [w * self.cache.page_size for w, g in zip(widths, paged)
                               if g.need.window is None])
            host = NoHostValues()
        ctx = StepContext(
            tokens=tokens, requests=requests, token_ids=on_device("token_ids"),
            positions=on_device("positions"), token_request=on_device("token_request"),
            request_start=on_device("request_start"), history=on_device("history"),
            max_portion=max_portion, max_context=max_context, views=views, host=host,
            replayable=captured is not None and self.use_graphs, leading_single=singles)

        device_fed = any(e.from_device for e in entries)

        def run():
            if device_fed:
                self.ops.resolve_tokens(ctx.token_ids, on_device("token_source"), self.published)
            residual, delta = self.model.forward(ctx)
            if not wanted:
                return None
            logits = self.model.logits(residual, delta,
                                       None if every_row else on_device("rows")[:wanted])
            if (greedy or draw is not None) and loop is None:
                if draw is not None:
                    chosen, _ = self.ops.sample(
                        logits, on_device("draw_temperature").view(torch.float32),
                        on_device("draw_top_k"), on_device("draw_top_p").view(torch.float32),
                        on_device("draw_seed").view(torch.int64), on_device("draw_step"))
                else:
                    chosen = self.ops.argmax(logits)
                report = self.ops.publish_tokens(chosen, on_device("want_index")[:wanted],
                                                 self.published)
                return logits, chosen, report
            return logits

        if loop is not None:
            return self._run_loop(captured, run, ctx, entries, *loop)
        if captured is None:
            logits = run()
        else:
            logits = self._run_captured(captured, run)
        self.last_greedy = self.last_report = None
        if isinstance(logits, tuple):
            logits, chosen, report = logits
            self.last_greedy = chosen[:real_wanted]
            # tokens of all wanted rows (fillers' after the real ones), then the error flag
            self.last_report = report
        if logits is not None:
            logits = logits[:real_wanted] if real_wanted else None
        for entry in entries:
            self.cache.advance(entry.request_id, len(entry.tokens))
        self.steps += 1
        self.last_shape = (requests, tokens)
        return logits

    def _run_loop(self, captured, run, ctx, entries, steps, record, events=None) -> torch.Tensor:
        if captured.counter is None:
            captured.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        captured.counter.zero_()
        captured.record = record

        def one_step():
            chosen = self.ops.argmax(run())
            # the graph may outlive this call's record; it always writes to captured.record
            self.ops.decode_advance(chosen, ctx.token_ids, ctx.positions, ctx.history,
                                    captured.record_buffer(record), captured.counter)

        done = 0
        if events is not None:
            events[0].record()
        if captured.graph is None or not self.use_graphs:
            one_step()
            done = 1
            captured.uses += 1
        if done < steps and self.use_graphs and captured.graph is None:
            captured.graph = self._capture(one_step)[0]
        for _ in range(done, steps):
            if captured.graph is not None:
                captured.graph.replay()
                self.graph_replays += 1
            else:
                one_step()
        if events is not None:
            events[1].record()
        out = captured.record_buffer(record)[:steps].clone()
        for entry in entries:
            self.cache.advance(entry.request_id, steps)
        self.steps += steps
        self.last_shape = (len(entries), len(entries))
        return out

    def _fill(self, singles: int, others: int, other_tokens: int, wanted: int):
        """Fillers that round a step's shape up to the next bucket: how many single-token
        requests after the leading ones, how many other requests with how many tokens between
        them, and how many wanted rows. ``singles``: leading requests that bring one token;
        ``others``: the requests after them, with ``other_tokens`` tokens together. A filler
        request brings at least one token, and filler tokens belong to a filler request. A
        decode-only step of up to ``request_bucket`` requests stays as it is."""
        up = lambda value, to: -(-value // to) * to
        bucket = self.request_bucket
        fill_wanted = up(wanted, bucket) - wanted if wanted else 0
        if others == 0:
            if singles <= bucket:
                return 0, 0, 0, 0
            return up(singles, bucket) - singles, 0, 0, fill_wanted
        fill_singles = up(singles, bucket) - singles
        step = self.token_bucket if other_tokens > 128 else 16
        to_others, to_tokens = up(others, 2), up(other_tokens, step)
        if to_tokens > other_tokens and to_others == others:
            to_others += 2
        while to_tokens - other_tokens < to_others - others:
            to_tokens += step
        return fill_singles, to_others - others, to_tokens - other_tokens, fill_wanted

    def _capture(self, run):
        """Records ``run`` into a CUDA graph; returns (graph, what run returned). A model whose
        parts all declare themselves capturable must be: a failure here is an error of a part
        (it synchronised, or read host values), and is raised, not hidden."""
        graph = torch.cuda.CUDAGraph()
        self.graph_captures += 1
        torch.cuda.current_stream(self.device).synchronize()
        reserved = torch.cuda.memory_reserved(self.device)
        try:
            with torch.cuda.graph(graph):
                result = run()
            # a graph keeps a memory pool of its own (its activations and logits): count what the
            # capture made the allocator reserve, so that it can be set against the cache's budget
            self.graph_memory_bytes += max(torch.cuda.memory_reserved(self.device) - reserved, 0)
        except Exception as error:
            torch.cuda.synchronize(self.device)
            raise RuntimeError(
                f"a step could not be captured as a CUDA graph ({error}); a part that "
                "synchronises or reads host values must set `capturable = False`") from error
        return graph, result

    def _forget_old_portion_graphs(self, newest: tuple) -> None:
        """A captured step keeps its activations' memory: of the shapes with portions only the
        ``portion_graphs`` most recently met are kept."""
        self._portion_keys = [k for k in self._portion_keys if k != newest] + [newest]
        while len(self._portion_keys) > self.portion_graphs:
            self._graphs.pop(self._portion_keys.pop(0), None)

    def _forget_old_decode_graphs(self, newest: tuple) -> None:
        """The same for decode-only shapes (batch sizes, table widths, greedy or sampled,
        device-fed or not): the ``decode_graphs`` most recently used are kept."""
        self._decode_keys = [k for k in self._decode_keys if k != newest] + [newest]
        while len(self._decode_keys) > self.decode_graphs:
            self._graphs.pop(self._decode_keys.pop(0), None)

    def graph_stats(self) -> dict[str, int]:
        """How many steps are kept as graphs, and how often one was replayed."""
        kept = sum(1 for g in self._graphs.values() if g.graph is not None)
        return {"graphs": kept, "graph_shapes": len(self._graphs),
                "graph_replays": self.graph_replays, "graph_captures": self.graph_captures,
                "graph_memory_bytes": self.graph_memory_bytes}

    def _run_captured(self, captured: _DecodeGraph, run, eager_uses: int = 1):
        """Steps of one shape: the first ``eager_uses`` run eagerly, the next is captured as a
        CUDA graph and replayed, later ones replay it. The logits of a replay live in the
        graph's memory and are overwritten by the next replay of the same shape."""
        captured.uses += 1
        if captured.uses <= eager_uses or not self.use_graphs:
            return run()
        if captured.graph is None:
            captured.graph, captured.logits = self._capture(run)
        captured.graph.replay()
        self.graph_replays += 1
        return captured.logits
