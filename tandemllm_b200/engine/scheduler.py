"""The scheduler above the step function: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees, and decides what happens when pages run out.

Every step:
  1. running requests with one token pending (decoding) get their row first, oldest first;
  2. the rest of the token budget goes to running requests that still have prompt (or recomputed text) to
     feed, oldest first, in portions of at most `chunk_size` tokens; a portion may be as short as one token;
  3. if the pages these rows need are not free, the most recently admitted running request is preempted:
     its pages and slot go back, it returns to the FRONT of the waiting line with everything it has
     (prompt and generated tokens) still to feed, and is recomputed when it is admitted again; the step
     function gives the same logits for recomputed text as for the original, so its output is unchanged;
  4. waiting requests are admitted, oldest first, while a slot is free, budget is left, the pages of their
     first portion are free and, beside running requests, all the text they bring fits next to all the text
     those still have to feed; admission never preempts.
A request whose prompt plus `max_tokens` can never fit in the whole pool, or exceeds `max_model_len`, is
refused when it is added.

The reference's server does the parts of this it needs for one GPU turn at a time: fixed slots and a
bounded queue (server/slots.py:874, :1248), prompt chunks one request at a time (engine.py:588-600), decode
rows of several slots in one joint pass (serving.py:366-387), and on `PoolFull` the lane gives its pages
back, waits at the head of the line and re-prefills prompt plus text (server/app.py:9386-9440). Finishing
follows `generate_greedy` (engine/spec.py:150-199): a stop id, the token limit, or the window's end.

The scheduler only does bookkeeping against the cache manager's page accounts; it runs without a device.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from ..sampling.sampler import SamplingParams, repeating_pattern

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
PENDING = -1        # in a request's output: a token that a launched step is still computing


@dataclass
class Request:
    request_id: object
    prompt: list[int]
    params: SamplingParams
    output: list[int] = field(default_factory=list)
    num_computed: int = 0           # tokens already in the cache
    state: str = WAITING
    finish_reason: str | None = None
    preemptions: int = 0
    order: int = 0
    last_slot: int | None = None    # where in `output` the request's last token sits, once that is known
    no_repeat: object = None        # the no-repeat-n-gram rule's memory (`sampling.NoRepeatIndex`), made at the first draw
    stop_pattern: tuple | None = None   # the block whose repetition ended the request (`SamplingParams.max_pattern_size`)

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    def span(self, start: int, count: int) -> list[int]:
        """tokens[start:start + count] without putting the whole text together (a step of a long request asks for one)."""
        n, end = len(self.prompt), start + count
        if end <= n:
            return self.prompt[start:end]
        if start >= n:
            return self.output[start - n:end - n]
        return self.prompt[start:] + self.output[:end - n]

    @property
    def pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.num_computed


@dataclass
class Scheduled:
    request: Request
    start: int          # index of the first token fed this step
    count: int          # tokens fed this step
    samples: bool       # the portion ends at the request's last token: a new token is drawn from its last row
    slot: int = -1      # where in the request's output that token goes (set when the step is accounted)
    finishes: bool = False   # the request ends with this step


@dataclass
class SchedulerStats:
    steps: int = 0
    rows: int = 0
    prompt_rows: int = 0
    decode_rows: int = 0
    preemptions: int = 0
    finished: int = 0


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int, chunk_size: int,
                 max_model_len: int, stop_token_ids: tuple[int, ...] = ()):
        if max_num_batched_tokens < 1 or chunk_size < 1 or max_num_seqs < 1:
            raise ValueError("max_num_seqs, max_num_batched_tokens and chunk_size must be positive")
        self.cache = cache
        self.max_num_seqs = min(max_num_seqs, cache.max_requests)
        self.budget = max_num_batched_tokens
        self.chunk_size = chunk_size
        self.max_model_len = max_model_len
        self.stop_token_ids = tuple(stop_token_ids)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self.stats = SchedulerStats()
        self._order = 0

    # ---- requests in ----
    def add(self, request: Request) -> None:
        n = len(request.prompt)
        if n == 0:
            raise ValueError(f"request {request.request_id!r}: the prompt is empty")
        if n + 1 > self.max_model_len:
            raise ValueError(f"request {request.request_id!r}: a prompt of {n} tokens leaves no room within "
                             f"max_model_len {self.max_model_len}")
        most = min(n + request.params.max_tokens, self.max_model_len)
        ps = self.cache.page_size
        for g in self.cache.groups:
            span = most if g.need.window is None else min(most, g.need.window + self.chunk_size + ps)
            if -(-span // ps) > g.pool.num_pages:
                raise ValueError(f"request {request.request_id!r}: {most} tokens need {-(-span // ps)} pages, "
                                 f"the pool has {g.pool.num_pages}")
        request.order = self._order
        self._order += 1
        request.state = WAITING
        self.waiting.append(request)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step's batch ----
    def _pages_short(self, chosen: list[tuple[Request, int]]) -> bool:
        wants = [(r.request_id, r.num_computed + n) for r, n in chosen]
        return not self.cache.can_reserve(wants)

    def _whole_text_fits(self, newcomer: Request, chosen: list[tuple[Request, int]]) -> bool:
        """Whether the free pages cover what the running requests and `newcomer` need to feed all the text they have
        (a group with a window never holds more than its window, a portion and a page of one request)."""
        ps = self.cache.page_size
        totals = {id(q): (q, len(q.prompt) + len(q.output)) for q in self.running}
        totals[id(newcomer)] = (newcomer, len(newcomer.prompt) + len(newcomer.output))
        for g in self.cache.groups:
            need = 0
            for q, total in totals.values():
                table = g.tables.get(q.request_id, [])
                more = -(-total // ps) - len(table)
                if g.need.window is not None:
                    span = -(-(g.need.window + self.chunk_size + ps) // ps)
                    more = min(more, span - sum(1 for p in table if p >= 0))
                need += max(0, more)
            if need > g.pool.free:
                return False
        return True

    def _preempt(self, victim: Request) -> None:
        self.cache.free(victim.request_id)
        self.running.remove(victim)
        victim.num_computed = 0
        victim.state = WAITING
        victim.preemptions += 1
        self.waiting.appendleft(victim)
        self.stats.preemptions += 1

    def schedule(self) -> list[Scheduled]:
        budget = self.budget
        chosen: list[tuple[Request, int]] = []
        # 1. decode rows, 2. portions of running requests
        for want_decode in (True, False):
            for r in sorted(self.running, key=lambda q: q.order):
                if budget == 0:
                    break
                if (r.pending == 1) != want_decode or any(c is r for c, _ in chosen):
                    continue
                n = min(r.pending, self.chunk_size, budget)
                chosen.append((r, n))
                budget -= n
        # 3. pages: preempt the newest until what is left fits
        short = False
        while chosen and self._pages_short(chosen):
            short = True
            victim = max(self.running, key=lambda q: q.order)
            for c, n in chosen:
                if c is victim:
                    budget += n
            chosen = [(c, n) for c, n in chosen if c is not victim]
            self._preempt(victim)
        # 4. admissions; none in a step that ran short of pages
        while not short and self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            r = self.waiting[0]
            n = min(r.pending, self.chunk_size, budget)
            # Beside running requests a newcomer is let in only if all the text it has to feed fits next to all the
            # text they still have to feed: letting it in on the strength of its first portion alone would have them
            # fight for pages and recompute each other's prompts over and over.
            if self.running and not self._whole_text_fits(r, chosen):
                break
            self.cache.admit(r.request_id)
            if self._pages_short(chosen + [(r, n)]):
                self.cache.free(r.request_id)
                break
            self.waiting.popleft()
            r.state = RUNNING
            self.running.append(r)
            chosen.append((r, n))
            budget -= n
        out = [Scheduled(r, r.num_computed, n, r.num_computed + n == len(r.prompt) + len(r.output)) for r, n in chosen]
        if out:
            self.stats.steps += 1
            for s in out:
                self.stats.rows += s.count
                if s.count == 1 and s.samples and s.request.output:
                    self.stats.decode_rows += 1
                else:
                    self.stats.prompt_rows += s.count
        return out

    # ---- results in ----
    def advance(self, batch: list[Scheduled]) -> None:
        """Account what is known of a step as soon as it is launched: the rows are in the cache, every sampling
        entry has a token coming (a PENDING place in its output until `resolve` fills it), and a request that
        reaches its token limit or the window's end with that token leaves the running set now. The next step can
        be scheduled, and launched with the pending tokens fed on the device, before this one's tokens are read."""
        for s in batch:
            r = s.request
            r.num_computed += s.count
            if not s.samples:
                continue
            r.output.append(PENDING)
            s.slot = len(r.output) - 1
            if len(r.output) >= r.params.max_tokens:
                r.finish_reason = "length"
            elif len(r.prompt) + len(r.output) >= self.max_model_len:
                r.finish_reason = "max_model_len"
            if r.finish_reason:
                s.finishes = True
                r.last_slot = s.slot
                self._retire(r)

    def _retire(self, r: Request) -> None:
        r.state = FINISHED
        self.running.remove(r)
        self.cache.free(r.request_id)

    def resolve(self, batch: list[Scheduled], new_tokens: list[int]) -> list[Request]:
        """The step's tokens are here: `new_tokens` holds one per entry with `samples`, in batch order. Fills the
        pending places, ends a request on a stop id (dropping what a step launched ahead of this one added for it)
        and returns the requests that finished with this step."""
        done = []
        it = iter(new_tokens)
        for s in batch:
            if not s.samples:
                continue
            tok = int(next(it))
            r = s.request
            if (r.last_slot is not None and s.slot > r.last_slot) or s.slot >= len(r.output):
                continue        # the request ended with an earlier token (or was aborted): this row ran for nothing
            r.output[s.slot] = tok
            stops = r.params.stop_token_ids if r.params.stop_token_ids is not None else self.stop_token_ids
            pattern = None
            if r.params.stops_on_patterns and not s.finishes:
                tail = r.params.max_pattern_size * r.params.min_count          # no pattern reaches further back
                pattern = repeating_pattern(r.output[max(0, s.slot + 1 - tail):s.slot + 1], r.params.min_pattern_size,
                                            r.params.max_pattern_size, r.params.min_count)
            if (not r.params.ignore_eos and tok in stops) or pattern is not None:
                r.finish_reason, r.stop_pattern = "stop", pattern
                del r.output[s.slot + 1:]
                r.last_slot = s.slot
                if r.state != FINISHED:
                    self._retire(r)
                s.finishes = True
            if s.finishes:
                self.finished.append(r)
                self.stats.finished += 1
                done.append(r)
        return done

    def update(self, batch: list[Scheduled], new_tokens: list[int]) -> list[Request]:
        """Account a whole step at once: `advance`, then `resolve`. Returns the requests that finished."""
        self.advance(batch)
        return self.resolve(batch, new_tokens)

    def abort(self, request: Request) -> None:
        """Take a request out wherever it is; its pages and slot go back."""
        if request.state == RUNNING:
            self.running.remove(request)
            self.cache.free(request.request_id)
        elif request.state == WAITING:
            self.waiting.remove(request)
        request.state, request.finish_reason, request.last_slot = FINISHED, "aborted", -1
