"""Sampling options of a request, and the batched draw on the device.

Options and their meaning are the reference's (`Sampler`, engine/sample.py:103-131): `temperature` 0 is
greedy whatever the filters say (sample.py:134-141); otherwise logits / temperature, then `min_p`, then
`top_k`, then `top_p` (sample.py:172-199), then a draw. A draw is Gumbel-max with noise keyed by
(seed, sequence position) (sample.py:311-322), so a seeded request yields the same tokens whatever shares
its batch; a request without a seed takes one from the operating system when it is made (sample.py:164-169).

Before the choice a request's logits take its `logit_bias` and its repetition, presence and frequency
penalties, with the reference's meanings (`PenaltySpec` and `PenaltyState`, engine/penalty.py:44-67,
189-232, 320-331): the history that the penalties read is the prompt and every token generated since, kept
as one row of counts a request on the device.

One kernel launch draws for every row of a step (`kernels.ops.sample`); a step of greedy rows only uses
the argmax kernel; a step in which no request asks for penalties or a bias launches nothing more.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable

import torch

from ..kernels import ops


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: int | None = None
    max_tokens: int = 128           # new tokens at most
    stop_token_ids: tuple[int, ...] | None = None    # None: the model's own stop ids
    ignore_eos: bool = False
    repetition_penalty: float = 1.0     # seen tokens: negative logits times this, the others divided by it
    presence_penalty: float = 0.0       # seen tokens lose this once
    frequency_penalty: float = 0.0      # seen tokens lose this times their count
    logit_bias: dict[int, float] | None = None      # {token id: added logit}
    no_repeat_ngram_size: int = 0       # n >= 2: a token that would repeat an n-gram of the text so far loses NO_REPEAT_PENALTY
    max_pattern_size: int = 0           # > 0 with min_count >= 2: the request ends when its last tokens are one block of
    min_pattern_size: int = 1           # min_pattern_size..max_pattern_size tokens repeated min_count times
    min_count: int = 0

    def __post_init__(self) -> None:
        if self.temperature < 0.0 or self.temperature != self.temperature:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be at least 1, got {self.max_tokens}")
        if not self.repetition_penalty > 0.0:
            raise ValueError(f"repetition_penalty must be > 0, got {self.repetition_penalty}")
        if not -2.0 <= self.presence_penalty <= 2.0:
            raise ValueError(f"presence_penalty must be in [-2, 2], got {self.presence_penalty}")
        if not -2.0 <= self.frequency_penalty <= 2.0:
            raise ValueError(f"frequency_penalty must be in [-2, 2], got {self.frequency_penalty}")
        if self.no_repeat_ngram_size and self.no_repeat_ngram_size < 2:
            raise ValueError(f"no_repeat_ngram_size must be 0 or >= 2, got {self.no_repeat_ngram_size}")
        if self.max_pattern_size < 0 or self.min_pattern_size < 1 or self.min_count < 0:
            raise ValueError(f"pattern stop: sizes {self.min_pattern_size}..{self.max_pattern_size}, count {self.min_count}")
        if self.logit_bias:
            bias = {}
            for k, v in self.logit_bias.items():         # keys may be strings of digits, as they are in JSON
                try:
                    t, v = int(k), float(v)
                    whole = isinstance(k, str) or t == k
                except (TypeError, ValueError):
                    whole = False
                if not whole or t < 0 or v != v:
                    raise ValueError(f"logit_bias maps token ids to numbers, got {k!r}: {v!r}")
                if v:
                    bias[t] = v
            self.logit_bias = bias or None
        else:
            self.logit_bias = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def penalizes(self) -> bool:
        """Some rule reads the request's history: it needs a row of counts."""
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0

    @property
    def changes_logits(self) -> bool:
        return self.penalizes or self.logit_bias is not None or self.no_repeat_ngram_size > 0

    @property
    def stops_on_patterns(self) -> bool:
        return self.max_pattern_size > 0 and self.min_count >= 2

    def resolved_seed(self) -> int:
        """The request's seed as a 63-bit integer; an unseeded request draws one now."""
        if self.seed is None:
            self.seed = int.from_bytes(os.urandom(8), "little") >> 1
        return int(self.seed) & ((1 << 63) - 1)


NO_REPEAT_PENALTY = 4.0      # what a token that would repeat an n-gram loses (the reference's `mask_penalty`: finite, so
                             # that a token the model is sure of can still win and the rule never forces an early end)
NO_REPEAT_WINDOW = 2048      # the text the rule looks back over: when it grows past this, the older half is forgotten


class NoRepeatIndex:
    """The no-repeat-n-gram rule's memory for one request, on the host: the request's text (prompt and generated
    tokens) over a window, and for every run of n - 1 tokens in it the tokens that followed the run
    (engine/penalty.py:169-254 of the reference: `history`, `followers`, `_add`, `_index_history`, `_mask`)."""

    def __init__(self, n: int):
        self.n = int(n)
        self.history: list[int] = []
        self.followers: dict[tuple, set[int]] = {}
        self.seen = 0                # tokens of the request's text taken in so far

    def add(self, ids: list[int]) -> None:
        n, h = self.n, self.history
        old = len(h)
        h.extend(int(t) for t in ids)
        self.seen += len(ids)
        if len(h) > NO_REPEAT_WINDOW:
            del h[:len(h) - NO_REPEAT_WINDOW // 2]
            self.followers.clear()
            old = 0
        for i in range(max(n - 1, old), len(h)):
            self.followers.setdefault(tuple(h[i - (n - 1):i]), set()).add(h[i])

    def blocked(self) -> set[int]:
        """The tokens that followed the text's last n - 1 tokens somewhere before."""
        tail = tuple(self.history[-(self.n - 1):])
        return self.followers.get(tail, set())


def repeating_pattern(tokens: list[int], min_size: int, max_size: int, count: int) -> tuple[int, ...] | None:
    """The block of min_size..max_size tokens that the end of `tokens` repeats `count` times, the shortest such, or None
    (the reference's `PatternStop.observe`, engine/penalty.py:133-156: a generation that writes one short pattern over and
    over is ended, not steered)."""
    n = len(tokens)
    for size in range(max(1, min_size), max_size + 1):
        span = size * count
        if n < span:
            continue
        base = n - span
        block = tokens[base:base + size]
        if all(tokens[base + k * size:base + (k + 1) * size] == block for k in range(1, count)):
            return tuple(block)
    return None


@dataclass
class SampleRow:
    """One logits row's request as the sampler sees it. `position` is the index in the sequence of the token being
    drawn. The last three matter to a request with penalties only: `slot`, the request's row among the counts (its slot
    in the cache); `owner`, a value that no other request in that slot ever has; `history`, a call that returns the
    `position` tokens before the drawn one, made only when the request's counts have to be built (its first draw, and
    the first after it lost its place)."""
    params: SamplingParams
    position: int
    slot: int = -1
    owner: object = None
    history: Callable[[], list[int]] | None = None
    blocked: set[int] | None = None      # tokens that take the no-repeat penalty in this draw (`NoRepeatIndex.blocked`)


class Sampler:
    """Draws one token per logits row on the device. Rows are `SampleRow`s, or (params, position) pairs for requests
    without penalties. `slots` is how many requests can be live at a time: the rows of the count table, which is made
    when the first request with penalties draws."""

    # float32: temperature, top_p, min_p, repetition, presence, frequency | int32: top_k, position, slot | int64: seed
    FIELDS = 11

    def __init__(self, device, slots: int = 0):
        self.device = device
        self.slots = int(slots)
        self.counts: torch.Tensor | None = None     # int32 [slots, vocabulary]
        self._counted: dict[int, tuple] = {}        # slot -> (owner, tokens counted)
        self._cap = 0

    def _staging(self, n: int):
        """A pinned block and its device copy for n rows. Three pairs take turns, each waiting only for the copy that last
        read it, so that a step can be launched while the one before it still runs."""
        if n > self._cap:
            self._cap = max(64, 2 * n)
            self._hosts = [torch.empty(self.FIELDS * self._cap, dtype=torch.int32, pin_memory=True) for _ in range(3)]
            self._devs = [torch.empty(self.FIELDS * self._cap, dtype=torch.int32, device=self.device) for _ in range(3)]
            self._events = [None, None, None]
            self._turn = 0
        self._turn = (self._turn + 1) % 3
        if self._events[self._turn] is not None:
            self._events[self._turn].synchronize()
        return self._hosts[self._turn], self._devs[self._turn]

    def _count_history(self, row: SampleRow, vocab: int) -> None:
        """Makes the request's row of counts hold its `position` tokens, if it does not already."""
        if not 0 <= row.slot < self.slots:
            raise ValueError(f"a request with penalties needs a slot below {self.slots}, got {row.slot}")
        if self.counts is None:
            self.counts = torch.zeros(self.slots, vocab, dtype=torch.int32, device=self.device)
        if self._counted.get(row.slot) == (row.owner, row.position):
            return
        if row.history is None:
            raise ValueError("a request with penalties needs its history at its first draw")
        tokens = row.history()
        if len(tokens) != row.position or any(t < 0 for t in tokens):
            raise ValueError(f"history of {len(tokens)} tokens for a draw at position {row.position}")
        self.counts[row.slot].zero_()
        if tokens:
            staged = torch.tensor(tokens, dtype=torch.int32).pin_memory()
            ops.count_tokens(self.counts, staged.to(self.device, non_blocking=True), row.slot)

    def _bias(self, rows: list[SampleRow], vocab: int):
        """(begin, token, value) on the device for the rows' added logits; None when no row has any."""
        if not any(r.params.logit_bias or r.blocked for r in rows):
            return None
        begin, token, value = [0], [], []
        for r in rows:
            added = dict(r.params.logit_bias or {})
            if r.blocked and len(r.blocked) < vocab:        # (a rule that would take the whole vocabulary down is skipped)
                for t in r.blocked:
                    added[t] = added.get(t, 0.0) - NO_REPEAT_PENALTY
            for t, v in sorted(added.items()):
                if t >= vocab:
                    raise ValueError(f"logit_bias names token {t}; the vocabulary has {vocab}")
                token.append(t)
                value.append(v)
            begin.append(len(token))
        ints = torch.tensor(begin + token, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        vals = torch.tensor(value, dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
        return ints[:len(begin)], ints[len(begin):], vals

    def forget(self, slot: int) -> None:
        """The slot's request is gone: whoever draws from it next starts its counts anew."""
        self._counted.pop(slot, None)

    def __call__(self, logits: torch.Tensor, rows: list) -> torch.Tensor:
        """int32 [n] token ids for float32 logits [n, V]. Logits of requests with penalties or a bias are changed in place."""
        n, vocab = logits.shape
        if n != len(rows):
            raise ValueError(f"{n} logits rows for {len(rows)} requests")
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
        if n == 0:
            return out
        rows = [r if isinstance(r, SampleRow) else SampleRow(*r) for r in rows]
        greedy = all(r.params.greedy for r in rows)
        changed = any(r.params.penalizes or r.params.logit_bias or r.blocked for r in rows)
        if greedy and not changed:
            return ops.argmax(logits, out)
        counted = [r for r in rows if r.params.penalizes]
        for r in counted:
            self._count_history(r, vocab)
        host, dev = self._staging(n)
        c = self._cap
        f = host.view(torch.float32)
        seeds = host[9 * c:11 * c].view(torch.int64)
        for i, r in enumerate(rows):
            p = r.params
            f[i] = p.temperature
            f[c + i] = p.top_p
            f[2 * c + i] = p.min_p
            f[3 * c + i] = p.repetition_penalty
            f[4 * c + i] = p.presence_penalty
            f[5 * c + i] = p.frequency_penalty
            host[6 * c + i] = p.top_k
            host[7 * c + i] = r.position
            host[8 * c + i] = r.slot if p.penalizes else -1
            seeds[i] = p.resolved_seed() if not p.greedy else 0
        dev.copy_(host, non_blocking=True)
        event = self._events[self._turn] or torch.cuda.Event()
        event.record()
        self._events[self._turn] = event
        df = dev.view(torch.float32)
        slot = dev[8 * c:8 * c + n]
        if changed:
            ops.penalize(logits, self.counts if counted else None, slot, df[3 * c:3 * c + n], df[4 * c:4 * c + n],
                         df[5 * c:5 * c + n], self._bias(rows, vocab))
        if greedy:
            ops.argmax(logits, out)
        else:
            ops.sample(logits, df[0:n], dev[6 * c:6 * c + n], df[c:c + n], df[2 * c:2 * c + n],
                       dev[9 * c:11 * c].view(torch.int64)[:n], dev[7 * c:7 * c + n], out)
        if counted:
            ops.count_tokens(self.counts, out, slot)
            for r in counted:
                self._counted[r.slot] = (r.owner, r.position + 1)
        return out
