"""The engine against the plain implementation over ways of feeding the same tokens: each request alone and
whole; most of it in one step and the last 32 tokens one by one; in portions of changing size; mixed with
other requests on so few pages that they are used again; through `bin/trace_run` itself; long decoding; the
first tokens of a sequence; greedy and sampled generation through the Python entry point. In 32-bit and in
bfloat16, on tiny models that differ in every size and option (A and B; C has the head size and widths the
tensor-core kernels of the bfloat16 path take).

Tolerances. 32-bit: every logit within 1e-4 of the row's largest magnitude. bfloat16: within 3e-2. The one
allowed exception is a position whose routing is a near tie in the plain implementation: when the k-th and the
(k+1)-th expert score of some layer are closer than the precision's noise in those scores (1e-5 in 32-bit; 3e-2
in bfloat16, where activations carry errors of about a hundredth of their size), the engine may choose the other
expert, and that token's logits then differ by much more than rounding. The reference sets near ties aside the
same way when it compares engines (tools/lfm_check.py:100-125). Such positions must be few (a tenth at most),
and a position with a clear routing margin must be within the tolerance, unless an earlier position of its own request
was set aside (it attends to that position's keys and values): then it must pass the check below. A position set
aside is not left unchecked: the trace is replayed once more with the engine recording the experts it chose
(`StepFunction.trace`), the plain implementation is run again with exactly that choice forced in every layer and
at every position of the request, and the position must then be within the tolerance.
"""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import plain_lfm2 as P
from tests import tiny_configs as T
from tests import traces
from tests.helpers import random_model_weights, write_folder

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
NEAR_TIE = {"float32": 1e-5, "bfloat16": 3e-2}
LENGTHS = (150, 97, 33, 64, 129, 48, 16, 81)


class Case:
    """A tiny model, its folder in the precision's storage type, its requests and the plain logits."""

    def __init__(self, name: str, dtype: str, tmp):
        self.name, self.dtype = name, dtype
        self.cfg = T.CONFIGS[name]
        exact = dtype == "bfloat16"
        self.W = random_model_weights(self.cfg, T.SEEDS[name], T.STD[name], bf16_exact=exact)
        self.folder = write_folder(str(tmp / f"{name}-{dtype}"), self.cfg, self.W,
                                   torch.bfloat16 if exact else torch.float32)
        self.requests = {f"q{i}": T.long_tokens(name, n, seed=20 + i) for i, n in enumerate(LENGTHS)}
        self.ref, self.margin = {}, {}
        for rid, toks in self.requests.items():
            margins = []
            self.ref[rid] = P.forward(self.cfg, self.W, toks, margins=margins)
            # per position, the tightest routing margin (a model without a routed layer has none to be near)
            self.margin[rid] = torch.stack(margins).min(0).values if margins else torch.full((len(toks),), float("inf"))

    def engine(self, max_tokens: int, parallel: int = 4, block_size: int = 16, **kw):
        from tandemllm_b200.engine import Engine, EngineArgs
        self._engine_args = dict(max_tokens=max_tokens, parallel=parallel, block_size=block_size, **kw)
        return Engine.from_folder(self.folder, EngineArgs(dtype=self.dtype, max_len=4096, parallel=parallel,
                                                          block_size=block_size,
                                                          kv_blocks=-(-max_tokens // block_size), **kw))

    def replay(self, engine, trace, routes: dict | None = None) -> dict:
        """(request, position) -> logits row, running `trace` through the engine's step function. With `routes` (a
        dict) the steps are traced and routes[(request, layer)][position] gets the experts the engine chose."""
        from tandemllm_b200.engine import StepEntry
        got, fed = {}, {}
        if routes is not None:
            engine.step_function.trace = {}
        for s in trace:
            entries = []
            for e in s["entries"]:
                if not engine.cache.has(e["id"]):
                    engine.admit(e["id"])
                entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
            logits = engine.step(entries).cpu()
            if routes is not None:
                for prefix, ids in engine.step_function.trace.get("routes", []):
                    li, ids, r = int(prefix.split(".")[1]), ids.cpu(), 0
                    for e in s["entries"]:
                        base = fed.get(e["id"], 0)
                        for j in range(len(e["tokens"])):
                            routes.setdefault((e["id"], li), {})[base + j] = ids[r + j]
                        r += len(e["tokens"])
            k = 0
            for e in s["entries"]:
                base = fed.get(e["id"], 0)
                for w in e["want"]:
                    got[(e["id"], base + w)] = logits[k]
                    k += 1
                fed[e["id"]] = base + len(e["tokens"])
            assert k == logits.shape[0]
            for rid in s["end"]:
                engine.release(rid)
        engine.cache.check()
        self._last = (dict(self._engine_args), trace, id(got))
        return got

    def recheck_with_the_engines_routes(self, rerouted: list, what: str) -> int:
        """Replays the last trace with the engine recording its choice of experts, runs the plain implementation again
        with that choice forced, and holds the positions that were set aside to the tolerance. Returns how many."""
        args, trace, _ = self._last
        routes: dict = {}
        again = self.replay(self.engine(**{**args, "graph": False}), trace, routes)
        checked = 0
        for rid in sorted({r for r, _, _ in rerouted}):
            toks = self.requests[rid]
            layers = sorted({li for (r, li) in routes if r == rid})
            if any(len(routes[(rid, li)]) < len(toks) for li in layers):
                continue                    # the trace did not feed the whole request: nothing to force
            forced = {li: torch.stack([routes[(rid, li)][p] for p in range(len(toks))]) for li in layers}
            ref = P.forward(self.cfg, self.W, toks, forced_routes=forced)
            for r, pos, _ in rerouted:
                if r != rid:
                    continue
                err = float((again[(rid, pos)] - ref[pos]).abs().max() / ref[pos].abs().max())
                assert err <= TOL[self.dtype], (f"{what} [{self.name} {self.dtype}]: {rid} position {pos} differs by "
                                                f"{err:.3g} from the plain implementation run with the engine's own choice "
                                                f"of experts; tolerance {TOL[self.dtype]:.1g}")
                checked += 1
        return checked

    def compare(self, got: dict, what: str) -> None:
        worst, rerouted, downstream, first_bad = 0.0, [], [], None
        touched = set()             # requests in which an earlier position went the other way at a routing near tie
        for (rid, pos), row in sorted(got.items()):
            ref = self.ref[rid][pos]
            err = float((row - ref).abs().max() / ref.abs().max())
            if err <= TOL[self.dtype]:
                worst = max(worst, err)
            elif float(self.margin[rid][pos]) < NEAR_TIE[self.dtype]:
                rerouted.append((rid, pos, round(err, 3)))          # a routing near tie went the other way
                touched.add(rid)
            elif rid in touched:
                # its own routing is clear, but it reads (keys, values, conv state) what a rerouted earlier position of
                # its request left: no excuse by itself, it must pass the check with the engine's routes forced below
                downstream.append((rid, pos, round(err, 3)))
            elif first_bad is None:
                first_bad = (rid, pos, err, float(self.margin[rid][pos]))
        assert first_bad is None, (f"{what} [{self.name} {self.dtype}]: first wrong token is {first_bad[0]} position "
                                   f"{first_bad[1]} (page offset {first_bad[1] % 16}) with error {first_bad[2]:.3g} and "
                                   f"routing margin {first_bad[3]:.3g}; tolerance {TOL[self.dtype]:.1g}")
        assert len(rerouted) <= max(1, len(got) // 10), (f"{what} [{self.name} {self.dtype}]: {len(rerouted)} of {len(got)} "
                                                         f"positions differ as routing near ties: {rerouted[:8]}")
        can_recheck = getattr(self, "_last", (None, None, None))[2] == id(got)
        assert not downstream or can_recheck, (f"{what} [{self.name} {self.dtype}]: positions behind a rerouted one differ "
                                               f"and cannot be rechecked here: {downstream[:8]}")
        if rerouted and can_recheck:
            checked = self.recheck_with_the_engines_routes(rerouted + downstream, what)
            assert checked >= len(downstream), "every position behind a rerouted one was held to the forced-route run"
            print(f"{what} [{self.name} {self.dtype}]: {len(rerouted)} of {len(got)} positions set aside as routing near "
                  f"ties and {len(downstream)} behind them, {checked} held to the plain implementation with the engine's "
                  f"choice forced")


def greedy_like_plain(case, prompt, out) -> None:
    """Teacher-forced: every generated token is the plain implementation's argmax at its place, or so close to it
    that the precision cannot tell them apart. In 32-bit it must be the argmax itself unless the two logits are
    within the 32-bit tolerance."""
    seq = list(prompt)
    for tok in out:
        ref = P.forward(case.cfg, case.W, seq)[-1]
        best = int(ref.argmax())
        if tok != best:
            margin = float(ref[best] - ref[tok])
            assert margin <= 2 * TOL[case.dtype] * float(ref.abs().max()), (len(seq), tok, best, margin)
        seq.append(tok)


@pytest.fixture(scope="module", params=[("a", "float32"), ("b", "float32"), ("c", "float32"), ("a", "bfloat16"),
                                        ("b", "bfloat16"), ("c", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    return Case(request.param[0], request.param[1], tmp_path_factory.mktemp("models"))


def test_each_request_alone_and_whole(case):
    eng = case.engine(max_tokens=256)
    got = case.replay(eng, traces.whole(case.requests))
    assert len(got) == sum(LENGTHS)
    case.compare(got, "whole")
    assert eng.cache.groups[0].pool.reused > 0


def test_most_in_one_step_then_the_last_32_one_by_one(case):
    eng = case.engine(max_tokens=256)
    case.compare(case.replay(eng, traces.decoded_tail(case.requests, 32)), "decoded tail")


def test_portions_of_changing_size(case):
    eng = case.engine(max_tokens=256)
    case.compare(case.replay(eng, traces.portions(case.requests)), "portions")
    case.compare(case.replay(eng, traces.portions(case.requests, sizes=(2, 3, 2, 5))), "small portions")


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_mixed_requests_on_few_pages(case, seed):
    trace = traces.mixed(case.requests, live=4, seed=seed)
    assert traces.live_at_once(trace) == 4
    held = traces.tokens_held(trace, 64)
    assert held < sum(-(-n // 64) * 64 for n in LENGTHS), "the trace must not fit everything at once"
    eng = case.engine(max_tokens=held)
    got = case.replay(eng, trace)
    assert len(got) == sum(LENGTHS)
    case.compare(got, f"mixed (seed {seed})")
    pool = eng.cache.groups[0].pool
    assert pool.reused > 0 and pool.free == pool.num_pages


def test_pages_of_32_and_64_tokens(case):
    for page in (32, 64):
        trace = traces.mixed(case.requests, live=3, seed=5)
        eng = case.engine(max_tokens=traces.tokens_held(trace, 64), block_size=page)
        case.compare(case.replay(eng, trace), f"mixed with pages of {page}")


def test_long_decoding(case):
    """One token at a time from the first token on, across many page edges."""
    toks = case.requests["q0"]
    trace = [{"step": i, "entries": [{"id": "q0", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    eng = case.engine(max_tokens=192)
    case.compare(case.replay(eng, trace), "long decoding")


def test_decode_graph_equals_eager_bit_for_bit(case):
    """Decode steps replayed from CUDA graphs give the eager step's bits (the reference holds its decode graph to
    the same, tests/gpu/test_lfm2_moe_gpu.py:158-186), alone and with two requests decoding together."""
    reqs = {"q1": case.requests["q1"], "q5": case.requests["q5"]}
    trace = traces.decoded_tail({"q1": reqs["q1"]}, 40)
    both = [{"step": 0, "entries": [{"id": r, "tokens": t[:20], "want": []} for r, t in reqs.items()], "end": []}]
    both += [{"step": 1 + i, "entries": [{"id": r, "tokens": [t[20 + i]], "want": [0]} for r, t in reqs.items()], "end": []}
             for i in range(25)]
    for tr in (trace, both):
        with_graph = case.engine(max_tokens=256, graph=True)
        eager = case.engine(max_tokens=256, graph=False)
        a, b = case.replay(with_graph, tr), case.replay(eager, tr)
        assert with_graph.step_function.graph_replays > 10 and eager.step_function.graph_replays == 0
        assert a.keys() == b.keys()
        for key in a:
            assert torch.equal(a[key], b[key]), key
        case.compare(a, "decode from graphs")


def test_a_captured_graph_survives_the_growth_of_kept_buffers(case):
    """Seventeen requests decode from a captured graph; then thirty decode together, which outgrows the routing plan (and
    whatever else is kept between steps) that the graph of seventeen was captured with; then the seventeen decode on from
    the old graph. A buffer freed on growth would be written by that replay while it belongs to somebody else. Every step's
    logits equal the eager engine's bit for bit."""
    n_many = 30
    toks = {f"m{i}": T.long_tokens(case.name, 24, seed=300 + i) for i in range(n_many)}
    first = [{"step": 0, "entries": [{"id": r, "tokens": t[:8], "want": []} for r, t in toks.items()], "end": []}]
    pair = [f"m{i}" for i in range(17)]     # (seventeen: past the experts' form for a dozen rows, which has a plan of its own)
    trace, at = list(first), {r: 8 for r in toks}

    def decode(who):
        entries = [{"id": r, "tokens": [toks[r][at[r]]], "want": [0]} for r in who]
        for r in who:
            at[r] += 1
        trace.append({"step": len(trace), "entries": entries, "end": []})
    for _ in range(4):
        decode(pair)
    decode(list(toks))
    decode(list(toks))
    for _ in range(4):
        decode(pair)
    engines = [case.engine(max_tokens=n_many * 32, parallel=n_many, graph=g) for g in (True, False)]
    a, b = (case.replay(e, trace) for e in engines)
    assert engines[0].step_function.graph_replays >= 6
    if case.dtype == "bfloat16" and case.name == "b":       # 8 experts, top-3: 90 pairs in tiles of 16 outgrow the plan for 64
        moe = [l.feed_forward for l in engines[0].model.layers if hasattr(l.feed_forward, "num_experts")]
        assert any(p._outgrown for p in moe), "the plan of the graph of seventeen was outgrown by the step of thirty"
    assert a.keys() == b.keys()
    for key in a:
        assert torch.equal(a[key], b[key]), key


def test_contexts_longer_than_a_span_of_keys(case):
    """700 tokens: portions whose keys lie in several spans (the CUDA-core kernels cut keys into spans of 256, the
    tensor-core kernel splits contexts above 512 over its grid), then 60 tokens decoded one by one across span and
    page edges, eagerly and from graphs."""
    rid = "long"
    if rid not in case.ref:
        toks = T.long_tokens(case.name, 700, seed=77)
        margins = []
        case.requests[rid] = toks
        case.ref[rid] = P.forward(case.cfg, case.W, toks, margins=margins)
        case.margin[rid] = torch.stack(margins).min(0).values
    toks = case.requests[rid]
    trace, at = [], 0
    for n in (300, 250, 90):
        trace.append({"step": len(trace), "entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
        at += n
    while at < len(toks):
        trace.append({"step": len(trace), "entries": [{"id": rid, "tokens": [toks[at]], "want": [0]}], "end": []})
        at += 1
    try:
        for graph in (False, True):
            got = case.replay(case.engine(max_tokens=768, graph=graph), trace)
            assert len(got) == len(toks)
            case.compare(got, f"a context of 700 tokens (graphs {graph})")
    finally:
        for d in (case.requests, case.ref, case.margin):
            d.pop(rid, None)


def test_first_tokens_of_a_sequence(case):
    """A sequence shorter than the conv taps and than a page; and a first portion of one token."""
    eng = case.engine(max_tokens=128)
    for n in (1, 2, 3):
        trace = [{"step": 0, "entries": [{"id": "q1", "tokens": case.requests["q1"][:n], "want": list(range(n))}],
                  "end": ["q1"]}]
        case.compare(case.replay(eng, trace), f"first {n} tokens")
    toks = case.requests["q2"]
    trace = [{"step": 0, "entries": [{"id": "q2", "tokens": toks[:1], "want": [0]}], "end": []},
             {"step": 1, "entries": [{"id": "q2", "tokens": toks[1:2], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "q2", "tokens": toks[2:], "want": list(range(len(toks) - 2))}], "end": ["q2"]}]
    case.compare(case.replay(eng, trace), "1 + 1 + rest")


def test_wanting_nothing_and_wanting_some(case):
    toks = case.requests["q3"]
    eng = case.engine(max_tokens=128)
    from tandemllm_b200.engine import StepEntry
    eng.admit("x")
    out = eng.step([StepEntry("x", toks[:40], [])])
    assert tuple(out.shape) == (0, case.cfg["vocab_size"])
    out = eng.step([StepEntry("x", toks[40:], [0, len(toks) - 41])]).cpu()
    eng.release("x")
    case.compare({("q3", 40): out[0], ("q3", len(toks) - 1): out[1]}, "wanted places")


def test_trace_run_program(case, tmp_path):
    """The replay program itself, as a user runs it: a mixed trace on standard input, logits files out."""
    trace = traces.mixed(case.requests, live=4, seed=3)
    out = tmp_path / "out"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", case.folder, "--dtype", case.dtype,
           "--out", str(out), "--max-tokens", str(traces.tokens_held(trace, 64))]
    r = subprocess.run(cmd, input="\n".join(json.dumps(s) for s in trace) + "\n", capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.split("\n") if ln] == [f"done {s['step']}" for s in trace]
    got, fed, V = {}, {}, case.cfg["vocab_size"]
    for s in trace:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, V)
        k = 0
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = torch.from_numpy(rows[k].copy())
                k += 1
            fed[e["id"]] = base + len(e["tokens"])
        assert k == rows.shape[0]
    case.compare(got, "bin/trace_run")


def test_greedy_generation_through_the_entry_point(case):
    from tandemllm_b200.sampling import SamplingParams
    eng = case.engine(max_tokens=1024)
    prompts = T.prompts(case.name)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert len(out) == 16
        greedy_like_plain(case, prompt, out)


def test_steps_launched_ahead_end_on_stop_ids_like_steps_taken_one_by_one(case):
    """With `overlap` the step after a decode step is launched before its tokens are read. Requests that end on a
    stop id (found one step late), by their token limit (known beforehand) and while others go on must give the
    text, the reasons and the page accounts of an engine that takes one step at a time."""
    from tandemllm_b200.sampling import SamplingParams
    prompts = T.prompts(case.name)
    free_run = case.engine(max_tokens=1024, overlap=False).generate(
        prompts, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))
    # stop ids taken from the free-running text, so that requests end at different steps
    # (every other request gets a stop id that never comes, and ends by its token limit)
    absent = lambda out: next(t for t in range(case.cfg["vocab_size"]) if t not in out)
    stops = [[out[5 + 3 * i]] if i % 2 == 0 else [absent(out)] for i, out in enumerate(free_run)]
    params = [SamplingParams(temperature=0.0, max_tokens=12 + 4 * i, stop_token_ids=tuple(st))
              for i, st in enumerate(stops)]
    results = {}
    for overlap in (False, True):
        eng = case.engine(max_tokens=1024, overlap=overlap)
        reqs = [eng.add_request(p, SamplingParams(**vars(sp))) for p, sp in zip(prompts, params)]
        while eng.scheduler.has_unfinished():
            eng.run_step()
        results[overlap] = [(r.output, r.finish_reason) for r in reqs]
        assert all(t >= 0 for r in reqs for t in r.output)
        eng.cache.check()
        assert all(g.pool.free == g.pool.num_pages for g in eng.cache.groups) and not eng.scheduler.running
    if case.dtype == "float32":
        assert results[True] == results[False]
    for (out, reason), sp, free in zip(results[True], params, free_run):
        assert reason in ("stop", "length") and len(out) <= sp.max_tokens
        assert (out[-1] in sp.stop_token_ids) == (reason == "stop") and not set(out[:-1]) & set(sp.stop_token_ids)
        if case.dtype == "float32":
            assert out == free[:len(out)]
    assert {reason for _, reason in results[True]} == {"stop", "length"} or len(prompts) < 2


def test_sampled_generation_in_mixed_chunks_repeats_and_matches_the_plain_draws(case):
    """Temperature 0.7 with a fixed seed, prompts fed as chunks of 8 beside decode tokens: the same tokens whatever
    the batching, and each token is the plain implementation's keyed draw from the plain logits."""
    from tandemllm_b200.sampling import SamplingParams
    prompts = T.prompts(case.name)
    sp = dict(temperature=0.7, top_k=40, top_p=0.95, seed=1234, max_tokens=12, ignore_eos=True)
    a = case.engine(max_tokens=1024, chunk_size=8, max_batched_tokens=16).generate(prompts, SamplingParams(**sp))
    b = case.engine(max_tokens=1024, chunk_size=512, max_batched_tokens=2048, parallel=1).generate(prompts, SamplingParams(**sp))
    if case.dtype == "float32":
        assert a == b
    agree = 0
    for prompt, out in zip(prompts, a):
        seq = list(prompt)
        for tok in out:
            ref = P.forward(case.cfg, case.W, seq)[-1]
            agree += tok == P.sample(ref, 0.7, 40, 0.95, 0.0, seed=1234, position=len(seq))
            seq.append(tok)
    total = sum(len(o) for o in a)
    assert agree >= (total if case.dtype == "float32" else int(0.8 * total)), (agree, total)


def test_out_of_pages_preempts_and_the_text_is_unchanged(case):
    from tandemllm_b200.sampling import SamplingParams
    prompts = [case.requests[r][:n] for r, n in (("q0", 60), ("q1", 50), ("q4", 40))]
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    roomy = case.engine(max_tokens=1024, parallel=3)
    want = roomy.generate(prompts, sp)
    tight = case.engine(max_tokens=208, parallel=3)        # 13 pages for three requests that grow to 100, 90 and 80 tokens
    got = tight.generate(prompts, sp)
    assert tight.scheduler.stats.preemptions > 0
    if case.dtype == "float32":
        assert got == want
    for prompt, out in zip(prompts, got):
        greedy_like_plain(case, prompt, out)
    tight.cache.check()
    assert tight.cache.groups[0].pool.free == tight.cache.groups[0].pool.num_pages
