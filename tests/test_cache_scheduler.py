"""The cache manager's page accounts and the scheduler's decisions, on the host with a fake step function."""

import random

import pytest

from tandemllm_b200.cache import CacheManager, OutOfPages
from tandemllm_b200.engine.scheduler import Request, Scheduler
from tandemllm_b200.parts.base import PagedNeed, SlotNeed
from tandemllm_b200.sampling import SamplingParams

NEEDS = [SlotNeed((2, 8)), PagedNeed(2, 16), SlotNeed((2, 8)), PagedNeed(2, 16), PagedNeed(2, 16, window=40)]


def manager(pages=8, reqs=3, page=16, needs=NEEDS):
    return CacheManager(needs, num_pages=pages, max_requests=reqs, page_size=page, device=None)


def test_groups_by_need_and_pages_of_their_own():
    m = manager()
    assert len(m.groups) == 2
    assert m.groups[0].sites == [1, 3] and m.groups[0].need.window is None
    assert m.groups[1].sites == [4] and m.groups[1].need.window == 40
    assert m.groups[0].pool is not m.groups[1].pool


def test_reserve_free_and_reuse():
    m = manager()
    m.admit("a")
    m.reserve("a", 33)
    assert len(m.table(0, "a")) == 3 and m.groups[0].pool.free == 5
    m.reserve("a", 40)                       # still three pages
    assert len(m.table(0, "a")) == 3
    m.advance("a", 40)
    first = list(m.table(0, "a"))
    m.free("a")
    assert m.groups[0].pool.free == 8
    m.admit("b")
    m.reserve("b", 16)
    assert m.table(0, "b")[0] == first[-1], "the page freed last is handed out first"
    assert m.groups[0].pool.reused == 1
    m.check()


def test_all_or_nothing_and_double_free():
    m = manager(pages=4)
    m.admit("a")
    m.reserve("a", 48)
    m.admit("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 40)
    assert m.table(0, "b") == [] and m.groups[0].pool.free == 1
    assert not m.can_reserve([("b", 40)]) and m.can_reserve([("b", 16)])
    m.free("b")
    with pytest.raises(RuntimeError, match="not admitted"):
        m.free("b")
    with pytest.raises(RuntimeError, match="already admitted"):
        m.admit("a")
    m.admit("b"); m.admit("c")
    with pytest.raises(OutOfPages, match="slots"):
        m.admit("d")
    m.check()


def test_window_group_gives_pages_back_as_the_request_advances():
    m = manager(pages=8)
    m.admit("a")
    n = 0
    for step in (20, 30, 25, 40, 1, 1, 1):
        n += step
        m.reserve("a", n)
        m.advance("a", n)
        full, win = m.table(0, "a"), m.table(1, "a")
        assert len(full) == -(-n // 16) and all(p >= 0 for p in full) if n <= 128 else True
        first_needed = max(0, n - 40 + 1) // 16
        assert all(p == -1 for p in win[:first_needed]) and all(p >= 0 for p in win[first_needed:])
        m.check()
    assert m.groups[1].pool.used <= 4
    m.free("a")
    assert m.groups[1].pool.free == 8 and m.groups[0].pool.free == 8


def test_random_orders_never_lose_or_share_a_page():
    rng = random.Random(0)
    m = manager(pages=12, reqs=4)
    live = {}
    for i in range(3000):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{i}"
            m.admit(rid)
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            new = live[rid] + rng.choice([1, 1, 2, 7, 16, 33])
            if m.can_reserve([(rid, new)]):
                m.reserve(rid, new)
                m.advance(rid, new)
                live[rid] = new
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, new)
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check()
        slots = [m.slot_of(r) for r in live]
        assert len(set(slots)) == len(slots)
    assert m.groups[0].pool.reused > 0


# ------------------------------------------------------------------------------------------ scheduler
class FakeStep:
    """Stands in for the step function: reserves pages like the real one and 'samples' a token that depends
    only on the request's tokens so far, so recomputed requests must reproduce their text."""

    def __init__(self, cache):
        self.cache = cache
        self.batches = []

    def run(self, batch):
        self.batches.append([(s.request.request_id, s.start, s.count, s.samples) for s in batch])
        out = []
        for s in batch:
            rid = s.request.request_id
            assert self.cache.length_of(rid) == s.start, "a portion must start where the cache ends"
            self.cache.reserve(rid, s.start + s.count)
            self.cache.advance(rid, s.start + s.count)
            if s.samples:
                toks = s.request.tokens
                out.append((sum(toks) * 31 + len(toks)) % 97 + 4)
        return out


def drive(sched, fake, limit=10_000):
    n = 0
    while sched.has_unfinished():
        batch = sched.schedule()
        assert batch, "the scheduler stalled with work left"
        sched.update(batch, fake.run(batch))
        sched.cache.check()
        n += 1
        assert n < limit
    return n


def make(pages=64, reqs=4, budget=32, chunk=8, max_len=256, needs=None):
    cache = manager(pages=pages, reqs=reqs, needs=needs or NEEDS[:4])
    return Scheduler(cache, max_num_seqs=reqs, max_num_batched_tokens=budget, chunk_size=chunk, max_model_len=max_len,
                     stop_token_ids=(3,)), FakeStep(cache)


def req(rid, n, max_tokens=5, **kw):
    return Request(rid, list(range(10, 10 + n)), SamplingParams(max_tokens=max_tokens, **kw))


def test_prompts_are_cut_under_the_budget_and_decodes_come_first():
    sched, fake = make(budget=12, chunk=8)
    a, b = req("a", 20), req("b", 5)
    sched.add(a); sched.add(b)
    drive(sched, fake)
    assert fake.batches[0] == [("a", 0, 8, False), ("b", 0, 4, False)]
    # a request with one token pending goes first, whether that token is decoded text or the prompt's last
    assert fake.batches[1] == [("b", 4, 1, True), ("a", 8, 8, False)]
    assert fake.batches[2][0] == ("b", 5, 1, True) and fake.batches[2][1] == ("a", 16, 4, True)
    for batch in fake.batches:
        assert sum(c for _, _, c, _ in batch) <= 12
    assert len(a.output) == 5 and len(b.output) == 5 and a.finish_reason == "length"
    assert sched.cache.groups[0].pool.free == 64 and not sched.running and not sched.waiting


def test_admission_waits_for_a_slot_fifo():
    sched, fake = make(reqs=2)
    rs = [req(f"r{i}", 6, max_tokens=3) for i in range(5)]
    for r in rs:
        sched.add(r)
    drive(sched, fake)
    firsts = {}
    for i, batch in enumerate(fake.batches):
        assert len(batch) <= 2
        for rid, *_ in batch:
            firsts.setdefault(rid, i)
    assert [firsts[f"r{i}"] for i in range(5)] == sorted(firsts[f"r{i}"] for i in range(5))
    assert all(len(r.output) == 3 for r in rs)


def test_finishing_on_stop_id_length_and_window():
    sched, fake = make(max_len=12)
    a = req("a", 10, max_tokens=50)
    sched.add(a)
    drive(sched, fake)
    assert a.finish_reason == "max_model_len" and len(a.prompt) + len(a.output) == 12
    sched, fake = make()
    b = Request("b", [1], SamplingParams(max_tokens=50, stop_token_ids=(39,)))     # (1*31+1)%97+4 = 36, then ...
    sched.add(b)
    fake.run = lambda batch, f=fake.run: [39 if len(s.request.output) == 2 else t for s, t in zip(batch, f(batch))]
    drive(sched, fake)
    assert b.finish_reason == "stop" and b.output[-1] == 39 and len(b.output) == 3
    c = Request("c", [1], SamplingParams(max_tokens=4, stop_token_ids=(39,), ignore_eos=True))
    sched.add(c)
    drive(sched, fake)
    assert c.finish_reason == "length" and len(c.output) == 4


def test_two_steps_in_the_air_drop_the_row_behind_a_stop_id():
    """`advance` when a step is launched, `resolve` when its tokens are read, with the next step scheduled in
    between: a request that ends on a stop id loses the row launched ahead of the news, one that ends by its token
    limit never gets such a row, and the pages of both go back once."""
    sched, fake = make()
    a = Request("a", [1, 2], SamplingParams(max_tokens=50, stop_token_ids=(77,)))
    b = Request("b", [5], SamplingParams(max_tokens=3, ignore_eos=True))
    sched.add(a), sched.add(b)
    first = sched.schedule()
    fake.run(first)
    sched.advance(first)
    assert a.output == [-1] and b.output == [-1] and a.pending == 1
    ahead = sched.schedule()                                   # scheduled before the first step's tokens are known
    assert [(s.request.request_id, s.count) for s in ahead] == [("a", 1), ("b", 1)]
    fake.run(ahead)
    sched.advance(ahead)
    assert sched.resolve(first, [40, 41]) == [] and a.output == [40, -1] and b.output == [41, -1]
    third = sched.schedule()
    fake.run(third)
    sched.advance(third)                                       # b reaches its limit here: known without its token
    assert b.state == "finished" and b not in sched.running and not sched.cache.has("b")
    assert sched.resolve(ahead, [77, 42]) == [a]               # a's stop id: its row in `third` ran for nothing
    assert a.output == [40, 77] and a.finish_reason == "stop" and not sched.cache.has("a")
    assert sched.schedule() == []
    assert sched.resolve(third, [99, 43]) == [b] and b.output == [41, 42, 43] and b.finish_reason == "length"
    assert a.output == [40, 77] and sched.finished == [a, b] and not sched.has_unfinished()
    sched.cache.check()
    assert all(g.pool.free == g.pool.num_pages for g in sched.cache.groups)


def test_a_repeating_pattern_ends_a_request_also_with_a_step_in_the_air():
    """`max_pattern_size` / `min_pattern_size` / `min_count`: the request ends with the token that completes the last of
    `min_count` copies of a block, with reason "stop" and the block on record; shorter runs and other requests go on; a
    row launched ahead of the news ran for nothing."""
    sched, fake = make()
    a = Request("a", [1], SamplingParams(max_tokens=50, ignore_eos=True, max_pattern_size=2, min_pattern_size=2, min_count=3))
    b = Request("b", [2], SamplingParams(max_tokens=9, ignore_eos=True))
    sched.add(a), sched.add(b)
    text = [50, 7, 8, 7, 8, 9, 7, 8, 7, 8, 7, 8, 60, 61]          # 7 8 7 8 (twice) goes on; 7 8 7 8 7 8 ends it
    fake.run = lambda batch, f=fake.run: [text[len(s.request.output)] if s.request is a else t
                                          for s, t in zip(batch, f(batch)) if s.samples]
    drive(sched, fake)
    assert a.finish_reason == "stop" and a.stop_pattern == (7, 8) and a.output == text[:12]
    assert b.finish_reason == "length" and len(b.output) == 9 and b.stop_pattern is None
    # two steps in the air
    sched, fake = make()
    c = Request("c", [1], SamplingParams(max_tokens=50, ignore_eos=True, max_pattern_size=1, min_count=2))
    sched.add(c)
    first = sched.schedule(); fake.run(first); sched.advance(first)
    ahead = sched.schedule(); fake.run(ahead); sched.advance(ahead)
    assert sched.resolve(first, [44]) == []
    third = sched.schedule(); fake.run(third); sched.advance(third)
    assert sched.resolve(ahead, [44]) == [c] and c.output == [44, 44] and c.stop_pattern == (44,)
    assert sched.resolve(third, [45]) == [] and c.output == [44, 44] and not sched.cache.has("c")
    sched.cache.check()


def test_refused_at_the_door():
    sched, _ = make(pages=4, max_len=100)
    with pytest.raises(ValueError, match="empty"):
        sched.add(Request("e", [], SamplingParams()))
    with pytest.raises(ValueError, match="max_model_len"):
        sched.add(req("long", 100))
    with pytest.raises(ValueError, match="pages"):
        sched.add(req("big", 60, max_tokens=30))       # 90 tokens = 6 pages > 4


def test_out_of_pages_preempts_the_newest_and_recomputes_the_same_text():
    # plenty of pages: the text every request must produce
    sched, fake = make(pages=64, reqs=3, budget=64, chunk=16)
    want = {}
    for rid, n in (("a", 30), ("b", 28), ("c", 26)):
        r = req(rid, n, max_tokens=24)
        sched.add(r)
        want[rid] = r
    drive(sched, fake)
    # 8 pages of 16 tokens for three requests that grow to about 54 tokens each (4 pages each): they cannot all stay
    sched2, fake2 = make(pages=8, reqs=3, budget=64, chunk=16)
    got = {}
    for rid, n in (("a", 30), ("b", 28), ("c", 26)):
        r = req(rid, n, max_tokens=24)
        sched2.add(r)
        got[rid] = r
    drive(sched2, fake2)
    assert sched2.stats.preemptions > 0
    assert got["a"].preemptions == 0, "the oldest request is never the victim while others run"
    for rid in want:
        assert got[rid].output == want[rid].output, rid
    assert sched2.cache.groups[0].pool.free == 8 and sched2.cache.groups[0].pool.reused > 0
    # a preempted request went back to the front of the line with nothing computed
    starts = [(rid, s) for batch in fake2.batches for rid, s, c, _ in batch if s == 0]
    assert len(starts) > 3


def test_a_newcomer_waits_until_its_whole_text_fits_beside_the_running():
    """12 pages; two prompts of 150 tokens (10 pages each), portions of 16. Let in on the strength of its first portion,
    the second would fight the first for pages and both would be recomputed again and again; instead it waits until
    the first is done: no preemption, and every prompt token is fed once."""
    sched, fake = make(pages=12, reqs=4, budget=32, chunk=16, max_len=400)
    a, b, c = req("a", 150, max_tokens=4), req("b", 150, max_tokens=4), req("c", 20, max_tokens=4)
    for r in (a, b, c):
        sched.add(r)
    drive(sched, fake)
    assert sched.stats.preemptions == 0 and sched.stats.prompt_rows == 150 + 150 + 20
    first_b = next(i for i, batch in enumerate(fake.batches) if any(rid == "b" for rid, *_ in batch))
    last_a = max(i for i, batch in enumerate(fake.batches) if any(rid == "a" for rid, *_ in batch))
    assert first_b > last_a, "b (10 pages) cannot sit beside a (10 pages) in 12"
    # c's two pages do fit beside b's ten: it is let in while b still feeds its prompt
    first_c = next(i for i, batch in enumerate(fake.batches) if any(rid == "c" for rid, *_ in batch))
    last_b = max(i for i, batch in enumerate(fake.batches) if any(rid == "b" for rid, *_ in batch))
    assert first_c < last_b
    assert all(len(r.output) == 4 for r in (a, b, c))


def test_random_load_finishes_everything_with_few_pages():
    rng = random.Random(1)
    sched, fake = make(pages=10, reqs=4, budget=24, chunk=7, max_len=120)
    rs = []
    for i in range(25):
        r = req(f"r{i}", rng.randint(1, 60), max_tokens=rng.randint(1, 30))
        sched.add(r)
        rs.append(r)
    drive(sched, fake, limit=100_000)
    assert all(r.state == "finished" for r in rs)
    assert sched.cache.groups[0].pool.free == 10 and sched.stats.finished == 25


def test_abort_gives_everything_back():
    sched, fake = make()
    a, b = req("a", 20), req("b", 20)
    sched.add(a); sched.add(b)
    batch = sched.schedule()
    sched.update(batch, fake.run(batch))
    sched.abort(a)
    drive(sched, fake)
    assert a.finish_reason == "aborted" and b.finish_reason == "length"
    assert sched.cache.groups[0].pool.free == 64


def test_a_span_of_a_request_is_a_slice_of_its_whole_text():
    """`Request.span` (what a step takes, without joining prompt and output) against slicing the joined text: spans
    inside the prompt, inside the output, across the seam, empty and past the end."""
    rng = random.Random(5)
    for _ in range(50):
        r = Request("r", [rng.randrange(100) for _ in range(rng.randrange(0, 9))], SamplingParams())
        r.output = [rng.randrange(100) for _ in range(rng.randrange(0, 9))]
        whole = r.tokens
        for start in range(len(whole) + 2):
            for count in range(0, len(whole) + 2 - start):
                assert r.span(start, count) == whole[start:start + count], (r.prompt, r.output, start, count)
