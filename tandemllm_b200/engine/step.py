"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A batch may hold portions of prompts of any length beside single decoded tokens, cut anywhere. The step
runs only the tokens it is given: it reserves their pages, lays the batch out as flat rows with each
row's request and position, writes the batch's integers into one pinned buffer and copies it to the
device once (the reference stages its rows the same way, engine/models/lfm2_moe/engine.py:249-341),
runs the model, and returns the logits at the wanted places as float32 [wanted, vocab]. Afterwards each
request's length has moved by its tokens and windowed groups have given back what no later row reads.

The reference never mixes prompt chunks and decode rows in one pass (engine.py:353-365, :602); here they
are the same case, because every kernel takes rows with explicit request, position and tables.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.manager import CacheManager
from ..parts.base import StepContext


@dataclass
class StepEntry:
    """`request`: the key the request was admitted under. `tokens`: its next tokens. `want`: indices into
    `tokens` whose logits are returned (may be empty)."""
    request: object
    tokens: list[int]
    want: list[int]


class KernelFault(RuntimeError):
    """A kernel recorded an index outside what it was given (and skipped the access)."""


_STATUS = {1: "a token id outside the vocabulary", 2: "a key/value write to a position without a page",
           3: "a visible key without a page"}


class StepFunction:
    def __init__(self, model, cache: CacheManager, check_status: bool = True):
        self.model, self.cache = model, cache
        self.device = model.runtime.device
        self.check_status = check_status
        self._pinned = None
        self._device_ints = None
        self.steps = 0
        self.rows_run = 0

    def _buffers(self, n: int):
        """A pinned staging buffer that no copy in flight still reads, and the device buffer it is copied to.
        Three pinned buffers take turns; each waits for the event recorded after its last copy."""
        if self._pinned is None or self._pinned[0].numel() < n:
            cap = max(4096, 2 * n)
            torch.cuda.current_stream().synchronize()
            self._pinned = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(3)]
            self._events = [None, None, None]
            self._turn = 0
            self._device_ints = torch.empty(cap, dtype=torch.int32, device=self.device)
        self._turn = (self._turn + 1) % 3
        if self._events[self._turn] is not None:
            self._events[self._turn].synchronize()
        return self._pinned[self._turn], self._device_ints

    def _copied(self) -> None:
        ev = self._events[self._turn] or torch.cuda.Event()
        ev.record()
        self._events[self._turn] = ev

    def build(self, entries: list[StepEntry]) -> StepContext:
        """Reserve pages for the batch and stage its integers on the device (one host-to-device copy)."""
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
            from ..cache.manager import OutOfPages
            raise OutOfPages(f"the step's {sum(len(e.tokens) for e in entries)} tokens need more pages than are free")
        for req, new_len in wants:
            cache.reserve(req, new_len)

        B = len(entries)
        R = sum(len(e.tokens) for e in entries)
        n_out = sum(len(e.want) for e in entries)
        G = len(cache.groups)
        max_pages = max(1, cache.max_table_len([e.request for e in entries]))
        total = 3 * R + (B + 1) + B + n_out + G * B * max_pages
        pinned, dev = self._buffers(total)
        host = pinned.numpy()
        o_tok, o_pos, o_req = 0, R, 2 * R
        o_start = 3 * R
        o_slot = o_start + B + 1
        o_out = o_slot + B
        o_tab = o_out + n_out
        r = 0
        k = 0
        max_rows = max_ctx = 0
        for b, e in enumerate(entries):
            n = len(e.tokens)
            start = cache.length_of(e.request)
            host[o_tok + r:o_tok + r + n] = e.tokens
            host[o_pos + r:o_pos + r + n] = range(start, start + n)
            host[o_req + r:o_req + r + n] = b
            host[o_start + b] = r
            host[o_slot + b] = cache.slot_of(e.request)
            for w in e.want:
                host[o_out + k] = r + w
                k += 1
            for g in range(G):
                t = cache.table(g, e.request)
                base = o_tab + (g * B + b) * max_pages
                host[base:base + len(t)] = t
                host[base + len(t):base + max_pages] = -1
            r += n
            max_rows = max(max_rows, n)
            max_ctx = max(max_ctx, start + n)
        host[o_start + B] = R
        dev[:total].copy_(pinned[:total], non_blocking=True)
        self._copied()
        tables = [dev[o_tab + g * B * max_pages:o_tab + (g + 1) * B * max_pages].view(B, max_pages) for g in range(G)]
        return StepContext(
            n_rows=R, n_requests=B, token_ids=dev[o_tok:o_tok + R], positions=dev[o_pos:o_pos + R],
            req_of_row=dev[o_req:o_req + R], row_start=dev[o_start:o_start + B + 1], state_slot=dev[o_slot:o_slot + B],
            block_tables=tables, out_rows=dev[o_out:o_out + n_out], n_out=n_out, max_rows_per_request=max_rows,
            max_context=max_ctx,
            host={"row_start": [int(x) for x in host[o_start:o_start + B + 1]],
                  "start_pos": [cache.length_of(e.request) for e in entries],
                  "slots": [cache.slot_of(e.request) for e in entries]})

    def run(self, entries: list[StepEntry]) -> torch.Tensor:
        """Logits float32 [wanted, vocab] in the order of the entries and of their `want`."""
        if not entries:
            return torch.empty(0, self.model.vocab_size, dtype=torch.float32, device=self.device)
        step = self.build(entries)
        logits = self.model.forward(step, self.cache.site_cache)
        for e in entries:
            self.cache.advance(e.request, self.cache.length_of(e.request) + len(e.tokens))
        self.steps += 1
        self.rows_run += step.n_rows
        if self.check_status:
            self.raise_on_fault()
        return logits

    def raise_on_fault(self) -> None:
        code = int(self.model.runtime.status.item())
        if code:
            self.model.runtime.status.zero_()
            raise KernelFault(f"a kernel recorded {_STATUS.get(code, f'status {code}')} and skipped the access")
