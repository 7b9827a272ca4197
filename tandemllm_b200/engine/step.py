"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A batch may hold portions of prompts of any length beside single decoded tokens, cut anywhere. The step
runs only the tokens it is given: it reserves their pages, lays the batch out as flat rows with each
row's request and position, writes the batch's integers into one pinned buffer and copies it to the
device once (the reference stages its rows the same way, engine/models/lfm2_moe/engine.py:249-341),
runs the model, and returns the logits at the wanted places as float32 [wanted, vocab]. Afterwards each
request's length has moved by its tokens and windowed groups have given back what no later row reads.

The reference never mixes prompt chunks and decode rows in one pass (engine.py:353-365, :602); here they
are the same case, because every kernel takes rows with explicit request, position and tables.

Decode-only steps (every request brings one token and wants its logits) can run from CUDA graphs, as the
reference replays one graph per decode token (engine.py:745-794): a graph is captured per batch size,
block-table width and context bucket the first time that shape has run eagerly, and replayed afterwards
from the same staged integers. The kernels and their order are the eager step's own. Context buckets grow
with the context (an eighth of the context's power of two, at least 1024 tokens), so a request that decodes
from 1 to 128k tokens passes through a few dozen of them, and at most `max_graphs` graphs are kept: beyond
that the least recently replayed one is dropped (at a moment when the stream is idle anyway, just before a
new one is captured).
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass

import numpy as np
import torch

from ..cache.manager import CacheManager, OutOfPages
from ..kernels import ops
from ..parts.base import StepContext
from ..settings import SETTINGS


@dataclass
class StepEntry:
    """`request`: the key the request was admitted under. `tokens`: its next tokens. `want`: indices into
    `tokens` whose logits are returned (may be empty)."""
    request: object
    tokens: list[int]
    want: list[int]


class KernelFault(RuntimeError):
    """A kernel recorded an index outside what it was given (and skipped the access), or gave up a bounded wait."""


_STATUS = {1: "a token id outside the vocabulary", 2: "a key/value write to a position without a page",
           3: "a visible key without a page", 4: "an attention tile with more rows than its kernel takes",
           5: "a plan tile with more rows than its kernel takes", 11: "a pipeline wait that ran out in a tensor-core kernel"}

CONTEXT_BUCKET = 1024       # the smallest context bucket of a decode graph


def context_bucket(longest: int) -> int:
    """The context a decode graph is captured for when its longest request holds `longest` tokens: the next
    multiple of g, g being an eighth of the power of two at or below `longest` and at least CONTEXT_BUCKET. A graph
    then serves contexts at most an eighth shorter than the one its kernels' grids were sized for, and contexts up to
    2^n fall into 8 buckets an octave."""
    g = CONTEXT_BUCKET
    while g * 16 <= longest:
        g *= 2
    return -(-longest // g) * g


class _Staging:
    """Three pinned buffers that take turns, so that a buffer is rewritten only after the copy that read it."""

    def __init__(self, cap: int):
        self.cap = cap
        self.buffers = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(3)]
        self.events = [None, None, None]
        self.turn = 0

    def next(self) -> torch.Tensor:
        self.turn = (self.turn + 1) % 3
        if self.events[self.turn] is not None:
            self.events[self.turn].synchronize()
        return self.buffers[self.turn]

    def copied(self) -> None:
        ev = self.events[self.turn] or torch.cuda.Event()
        ev.record()
        self.events[self.turn] = ev


class _DecodeGraph:
    """One captured decode step: its device integers, its context, the graph and the logits it writes."""

    def __init__(self, dev: torch.Tensor, step: StepContext):
        self.dev, self.step = dev, step
        self.graph: ops.DeviceGraph | None = None
        self.kernels = 0
        self.logits: torch.Tensor | None = None


class StepFunction:
    def __init__(self, model, cache: CacheManager, check_status: bool = True, use_graphs: bool = False,
                 max_graph_batch: int = 64, max_graphs: int | None = None):
        self.model, self.cache = model, cache
        self.device = model.runtime.device
        self.check_status = check_status
        self.use_graphs = use_graphs
        self.max_graph_batch = max_graph_batch
        self._staging: _Staging | None = None
        self._device_ints = None
        self._graphs: OrderedDict[tuple, _DecodeGraph] = OrderedDict()      # least recently used first
        self._graph_pool = None
        self._capture_stream = None
        self.max_graphs = max(1, max_graphs if max_graphs is not None else SETTINGS.get_int("GRAPHS"))
        self.graphs_dropped = 0
        self.trace: dict | None = None      # when a dict: every step runs eagerly and its parts may record into it
        self.steps = 0
        self.rows_run = 0
        self.graph_replays = 0
        self.last_from_graph = False        # whether the last step was a graph replay

    # ---- laying a batch out ----
    def _pinned(self, n: int) -> torch.Tensor:
        if self._staging is None or self._staging.cap < n:
            torch.cuda.current_stream().synchronize()
            self._staging = _Staging(max(4096, 2 * n))
        return self._staging.next()

    def _reserve(self, entries: list[StepEntry]) -> None:
        cache = self.cache
        wants = []
        for e in entries:
            if not e.tokens:
                raise ValueError(f"request {e.request!r} brings no tokens to this step")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"request {e.request!r}: wanted place {w} is not among its {len(e.tokens)} tokens")
            wants.append((e.request, cache.length_of(e.request) + len(e.tokens)))
        if len({e.request for e in entries}) != len(entries):
            raise ValueError("a request appears twice in one step")
        if not cache.can_reserve(wants):
            raise OutOfPages(f"the step's {sum(len(e.tokens) for e in entries)} tokens need more pages than are free")
        for req, new_len in wants:
            cache.reserve(req, new_len)

    @staticmethod
    def _layout(B: int, R: int, n_out: int, G: int, max_pages: int) -> dict:
        o = {"tok": 0, "pos": R, "req": 2 * R, "start": 3 * R}
        o["slot"] = o["start"] + B + 1
        o["out"] = o["slot"] + B
        o["tab"] = o["out"] + n_out
        o["total"] = o["tab"] + G * B * max_pages
        return o

    def _fill(self, host, o: dict, entries: list[StepEntry], max_pages: int) -> tuple[int, int]:
        """Write the batch's integers into `host` (a numpy view) at layout `o`; returns (most rows of a request,
        longest context after the step)."""
        cache = self.cache
        B, G = len(entries), len(cache.groups)
        r = k = max_rows = max_ctx = 0
        for b, e in enumerate(entries):
            n = len(e.tokens)
            start = cache.length_of(e.request)
            host[o["tok"] + r:o["tok"] + r + n] = e.tokens
            host[o["pos"] + r:o["pos"] + r + n] = range(start, start + n)
            host[o["req"] + r:o["req"] + r + n] = b
            host[o["start"] + b] = r
            host[o["slot"] + b] = cache.slot_of(e.request)
            for w in e.want:
                host[o["out"] + k] = r + w
                k += 1
            for g in range(G):
                t = cache.table_array(g, e.request)
                base = o["tab"] + (g * B + b) * max_pages
                host[base:base + len(t)] = t
                host[base + len(t):base + max_pages] = -1
            r += n
            max_rows = max(max_rows, n)
            max_ctx = max(max_ctx, start + n)
        host[o["start"] + B] = r
        return max_rows, max_ctx

    def _fill_decode(self, host, o: dict, entries: list[StepEntry], max_pages: int) -> None:
        """`_fill` for a step of one token a request whose logits are all wanted: whole columns at a time."""
        cache = self.cache
        B, G = len(entries), len(cache.groups)
        reqs = [e.request for e in entries]
        count = np.arange(B + 1, dtype=np.int32)
        host[o["tok"]:o["tok"] + B] = [e.tokens[0] for e in entries]
        host[o["pos"]:o["pos"] + B] = [cache.length_of(r) for r in reqs]
        host[o["req"]:o["req"] + B] = count[:B]
        host[o["start"]:o["start"] + B + 1] = count
        host[o["slot"]:o["slot"] + B] = [cache.slot_of(r) for r in reqs]
        host[o["out"]:o["out"] + B] = count[:B]
        tables = host[o["tab"]:o["tab"] + G * B * max_pages].reshape(G, B, max_pages)
        tables.fill(-1)
        for g in range(G):
            for b, r in enumerate(reqs):
                t = cache.table_array(g, r)
                tables[g, b, :t.shape[0]] = t

    def _context(self, dev: torch.Tensor, o: dict, B: int, R: int, n_out: int, max_pages: int, max_rows: int,
                 max_ctx: int, host_lists: dict) -> StepContext:
        if self.trace is not None:
            self.trace.clear()
        G = len(self.cache.groups)
        tables = [dev[o["tab"] + g * B * max_pages:o["tab"] + (g + 1) * B * max_pages].view(B, max_pages) for g in range(G)]
        return StepContext(
            n_rows=R, n_requests=B, token_ids=dev[o["tok"]:o["tok"] + R], positions=dev[o["pos"]:o["pos"] + R],
            req_of_row=dev[o["req"]:o["req"] + R], row_start=dev[o["start"]:o["start"] + B + 1],
            state_slot=dev[o["slot"]:o["slot"] + B], block_tables=tables, out_rows=dev[o["out"]:o["out"] + n_out],
            n_out=n_out, max_rows_per_request=max_rows, max_context=max_ctx, host=host_lists, trace=self.trace)

    def build(self, entries: list[StepEntry]) -> StepContext:
        """Reserve pages for the batch and stage its integers on the device (one host-to-device copy)."""
        self._reserve(entries)
        cache = self.cache
        B = len(entries)
        R = sum(len(e.tokens) for e in entries)
        n_out = sum(len(e.want) for e in entries)
        max_pages = max(1, cache.max_table_len([e.request for e in entries]))
        o = self._layout(B, R, n_out, len(cache.groups), max_pages)
        pinned = self._pinned(o["total"])
        if self._device_ints is None or self._device_ints.numel() < o["total"]:
            self._device_ints = torch.empty(max(4096, 2 * o["total"]), dtype=torch.int32, device=self.device)
        dev = self._device_ints
        host = pinned.numpy()
        max_rows, max_ctx = self._fill(host, o, entries, max_pages)
        dev[:o["total"]].copy_(pinned[:o["total"]], non_blocking=True)
        self._staging.copied()
        lists = {"row_start": [int(x) for x in host[o["start"]:o["start"] + B + 1]],
                 "start_pos": [cache.length_of(e.request) for e in entries],
                 "slots": [cache.slot_of(e.request) for e in entries]}
        return self._context(dev, o, B, R, n_out, max_pages, max_rows, max_ctx, lists)

    # ---- running ----
    def run(self, entries: list[StepEntry], feedback: tuple[torch.Tensor, list[int]] | None = None) -> torch.Tensor:
        """Logits float32 [wanted, vocab] in the order of the entries and of their `want`. `feedback` = (int32 token
        ids on the device, an index into them for every entry): each entry brings one token, and it is taken from
        there instead of from the entry (the step before this one may still be computing it)."""
        if not entries:
            return torch.empty(0, self.model.vocab_size, dtype=torch.float32, device=self.device)
        if feedback is not None and (len(feedback[1]) != len(entries) or any(len(e.tokens) != 1 for e in entries)):
            raise ValueError("tokens fed on the device: one token and one index for every entry")
        self.last_from_graph = False
        if (self.use_graphs and self.trace is None and len(entries) <= self.max_graph_batch
                and all(len(e.tokens) == 1 and e.want == [0] for e in entries)):
            logits = self._run_decode_graph(entries, feedback)
        else:
            step = self.build(entries)
            self._feed(step, feedback)
            logits = self.model.forward(step, self.cache.site_cache)
        for e in entries:
            self.cache.advance(e.request, self.cache.length_of(e.request) + len(e.tokens))
        self.steps += 1
        self.rows_run += sum(len(e.tokens) for e in entries)
        if self.check_status:
            self.raise_on_fault()
        return logits

    def _feed(self, step: StepContext, feedback) -> None:
        if feedback is None:
            return
        source, index = feedback
        if index == list(range(source.numel())):
            step.token_ids.copy_(source)
        else:
            step.token_ids.copy_(source[torch.tensor(index, dtype=torch.int64).to(self.device, non_blocking=True)])

    def _run_decode_graph(self, entries: list[StepEntry], feedback=None) -> torch.Tensor:
        """A decode-only step: eager the first time its shape is seen (and then captured), a graph replay after."""
        self._reserve(entries)
        cache = self.cache
        B = len(entries)
        pages = max(1, cache.max_table_len([e.request for e in entries]))
        width = 8
        while width < pages:
            width *= 2
        longest = max(cache.length_of(e.request) for e in entries) + 1
        ctx = context_bucket(longest)
        key = (B, width, ctx)
        o = self._layout(B, B, B, len(cache.groups), width)
        slot = self._graphs.get(key)
        if slot is not None:
            self._graphs.move_to_end(key)
        else:
            dev = torch.empty(o["total"], dtype=torch.int32, device=self.device)
            lists = {"row_start": list(range(B + 1)), "start_pos": None, "slots": None}
            slot = self._graphs[key] = _DecodeGraph(dev, self._context(dev, o, B, B, B, width, 1, ctx, lists))
        pinned = self._pinned(o["total"])
        self._fill_decode(pinned.numpy(), o, entries, width)
        slot.dev.copy_(pinned[:o["total"]], non_blocking=True)
        self._staging.copied()
        self._feed(slot.step, feedback)
        if slot.graph is not None:
            slot.graph.replay()
            self.graph_replays += 1
            self.last_from_graph = True
            ops.launches += slot.kernels
            return slot.logits
        # the first step of this shape runs eagerly (it also sizes every kept buffer); then the same calls are
        # captured for the steps that follow. Capturing launches nothing.
        logits = self.model.forward(slot.step, cache.site_cache)
        torch.cuda.current_stream().synchronize()
        while len(self._graphs) > self.max_graphs:
            # The stream is idle, so no replay of the dropped graph is running. Its logits go back to the graphs' shared
            # pool with it; a caller that still holds them from an earlier step has had them read (the stream is idle).
            self._graphs.popitem(last=False)
            self.graphs_dropped += 1
        # One memory pool for all the graphs of this step function: what a graph's kernels write between them lives there,
        # and a dropped graph's memory is used again by the next capture.
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.MemPool()
        graph = ops.DeviceGraph()
        before = ops.launches
        # Captured on a stream of its own, on the runtime API (`ops.DeviceGraph`; `torch.cuda.graph(...)` would also run
        # the garbage collector and hand every cached block back to the driver first: hundreds of milliseconds here, and
        # the steps after it pay for the blocks again. The stream is idle and the shapes were sized by the eager run.)
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device=self.device)
        current = torch.cuda.current_stream()
        self._capture_stream.wait_stream(current)
        with torch.cuda.stream(self._capture_stream):
            graph.capture_begin(pool=self._graph_pool)
            try:
                slot.logits = self.model.forward(slot.step, cache.site_cache)
            finally:
                graph.capture_end()
        current.wait_stream(self._capture_stream)
        slot.kernels = ops.launches - before        # kernels one replay runs; capturing ran none
        ops.launches = before
        slot.graph = graph
        return logits

    def drop_graphs(self) -> None:
        """Forget every captured graph (what a step runs has changed: the next decode steps run eagerly and are
        captured again)."""
        torch.cuda.current_stream().synchronize()
        self._graphs.clear()

    def raise_on_fault(self) -> None:
        code = int(self.model.runtime.status.item())
        if code:
            self.model.runtime.status.zero_()
            raise KernelFault(f"a kernel recorded {_STATUS.get(code, f'status {code}')} and skipped the access")
