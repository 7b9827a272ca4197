"""Repetition, presence and frequency penalties and added logits: the two kernels alone against the plain implementation, the
sampler's bookkeeping of a request's counts (built at the first draw, kept from then on, built again for another owner of
the slot), and generation through the scheduler on a cache so small that requests are preempted and recomputed, every
token held to the plain implementation run on the text so far."""

import pytest
import torch

from tests import plain_lfm2 as P
from tests import tiny_configs as T
from tests.helpers import random_model_weights, write_folder

pytestmark = pytest.mark.gpu
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


def _histories(g, rows, vocab, longest):
    out = []
    for _ in range(rows):
        n = int(torch.randint(1, longest, (1,), generator=g))
        few = torch.randint(0, vocab, (max(2, n // 4),), generator=g)         # drawn from a few tokens: counts above one
        out.append(few[torch.randint(0, few.numel(), (n,), generator=g)].tolist())
    return out


@pytest.mark.parametrize("vocab", [1003, 65536 + 24])
def test_penalty_kernel_matches_the_plain_rule_row_by_row(vocab):
    from tandemllm_b200.kernels import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(vocab)
    rows, slots = 6, 9
    logits = torch.randn(rows, vocab, generator=g) * 4
    hist = _histories(g, rows, vocab, 300)
    slot = [7, -1, 0, 3, -1, 8]                     # two rows without penalties, one of them with a bias
    rep = [1.3, 1.0, 1.0, 0.7, 1.0, 1.15]
    pres = [0.0, 0.0, 1.5, -0.5, 0.0, 0.25]
    freq = [0.0, 0.0, 0.6, 0.0, 0.0, -0.125]
    bias = [None, {5: 3.5, vocab - 1: -7.0}, {hist[2][0]: 2.0}, None, None, {0: -1.0, 17: 4.0, hist[5][3]: 0.5}]
    counts = torch.zeros(slots, vocab, dtype=torch.int32, device=dev)
    counts[1] = 5                                   # a row that nobody names: its counts must not matter
    for r in range(rows):
        if slot[r] >= 0:
            ops.count_tokens(counts, torch.tensor(hist[r], dtype=torch.int32, device=dev), slot[r])
    for r in range(rows):
        if slot[r] >= 0:
            assert torch.equal(counts[slot[r]].cpu().long(), torch.bincount(torch.tensor(hist[r]), minlength=vocab))
    begin, token, value = [0], [], []
    for b in bias:
        for t, v in sorted((b or {}).items()):
            token.append(t); value.append(v)
        begin.append(len(token))
    out = logits.to(dev)
    ops.penalize(out, counts, torch.tensor(slot, dtype=torch.int32, device=dev),
                 torch.tensor(rep, device=dev), torch.tensor(pres, device=dev), torch.tensor(freq, device=dev),
                 (torch.tensor(begin, dtype=torch.int32, device=dev), torch.tensor(token, dtype=torch.int32, device=dev),
                  torch.tensor(value, device=dev)))
    out = out.cpu()
    for r in range(rows):
        want = P.penalize(logits[r], hist[r] if slot[r] >= 0 else [], rep[r], pres[r], freq[r], bias[r])
        assert (out[r] - want).abs().max() <= 2e-6 * want.abs().max(), r
        if slot[r] < 0 and bias[r] is None:
            assert torch.equal(out[r], logits[r])
    # without any bias, and without any counts: the other two forms of the call
    plain_rows = logits.to(dev)
    ops.penalize(plain_rows, counts, torch.tensor(slot, dtype=torch.int32, device=dev), torch.tensor(rep, device=dev),
                 torch.tensor(pres, device=dev), torch.tensor(freq, device=dev))
    for r in range(rows):
        want = P.penalize(logits[r], hist[r] if slot[r] >= 0 else [], rep[r], pres[r], freq[r])
        assert (plain_rows[r].cpu() - want).abs().max() <= 2e-6 * want.abs().max(), r
    only_bias = logits[:2].to(dev)
    none = torch.full((2,), -1, dtype=torch.int32, device=dev)
    ones, zeros = torch.ones(2, device=dev), torch.zeros(2, device=dev)
    ops.penalize(only_bias, None, none, ones, zeros, zeros,
                 (torch.tensor([0, 0, 1], dtype=torch.int32, device=dev), torch.tensor([9], dtype=torch.int32, device=dev),
                  torch.tensor([2.5], device=dev)))
    want = logits[:2].clone()
    want[1, 9] += 2.5
    assert torch.equal(only_bias.cpu(), want)


def test_counting_with_a_slot_for_every_token_passes_over_rows_without_one():
    from tandemllm_b200.kernels import ops
    dev = torch.device("cuda:0")
    counts = torch.zeros(4, 77, dtype=torch.int32, device=dev)
    tokens = torch.tensor([5, 76, 5, 0, 12], dtype=torch.int32, device=dev)
    slot = torch.tensor([2, 0, 2, -1, 3], dtype=torch.int32, device=dev)
    ops.count_tokens(counts, tokens, slot)
    ops.count_tokens(counts, tokens, slot)
    want = torch.zeros(4, 77, dtype=torch.int32)
    want[2, 5], want[0, 76], want[3, 12] = 4, 2, 2
    assert torch.equal(counts.cpu(), want)


def test_sampler_builds_a_requests_counts_once_and_again_for_the_slots_next_owner():
    from tandemllm_b200.sampling import Sampler, SampleRow, SamplingParams
    dev = torch.device("cuda:0")
    vocab = 300
    g = torch.Generator().manual_seed(5)
    sampler = Sampler(dev, slots=3)
    pen = SamplingParams(frequency_penalty=-0.75, presence_penalty=0.5)       # the oftener seen, the likelier: counts matter
    plain = SamplingParams()
    hist = {"a": [4, 4, 9, 250, 4], "b": [1, 2, 3]}
    calls = []

    def history(name):
        def read():
            calls.append(name)
            return list(hist[name])
        return read

    for step in range(6):
        logits = torch.randn(3, vocab, generator=g)
        rows = [SampleRow(pen, len(hist["a"]), 2, "a", history("a")), SampleRow(plain, 40 + step),
                SampleRow(pen, len(hist["b"]), 0, "b", history("b"))]
        got = sampler(logits.to(dev), rows).tolist()
        want = [int(P.penalize(logits[0], hist["a"], presence=0.5, frequency=-0.75).argmax()), int(logits[1].argmax()),
                int(P.penalize(logits[2], hist["b"], presence=0.5, frequency=-0.75).argmax())]
        assert got == want, step
        hist["a"].append(got[0]); hist["b"].append(got[2])
    assert calls == ["a", "b"]                      # read at the first draw only
    for name, slot in (("a", 2), ("b", 0)):
        assert torch.equal(sampler.counts[slot].cpu().long(), torch.bincount(torch.tensor(hist[name]), minlength=vocab))
    # another request takes slot 2 at the very position the old one had reached; and "b" comes back after losing its place
    hist["c"] = list(range(100, 100 + len(hist["a"])))
    logits = torch.randn(2, vocab, generator=g)
    got = sampler(logits.to(dev), [SampleRow(pen, len(hist["c"]), 2, "c", history("c")),
                                   SampleRow(pen, len(hist["b"]), 1, ("b", "again"), history("b"))]).tolist()
    assert calls[2:] == ["c", "b"]
    assert got == [int(P.penalize(logits[0], hist["c"], presence=0.5, frequency=-0.75).argmax()),
                   int(P.penalize(logits[1], hist["b"], presence=0.5, frequency=-0.75).argmax())]
    with pytest.raises(ValueError, match="slot"):
        sampler(logits.to(dev)[:1], [SampleRow(pen, 3, 3, "d", lambda: [1, 2, 3])])
    with pytest.raises(ValueError, match="history"):
        sampler(logits.to(dev)[:1], [SampleRow(pen, 3, 1, "d", lambda: [1, 2])])
    with pytest.raises(ValueError, match="logit_bias"):
        sampler(logits.to(dev)[:1], [SampleRow(SamplingParams(logit_bias={vocab: 1.0}), 3)])


def _params(i, new_tokens, prompt):
    from tandemllm_b200.sampling import SamplingParams
    common = dict(max_tokens=new_tokens, ignore_eos=True)
    kinds = [
        dict(repetition_penalty=1.8),
        dict(presence_penalty=-1.0, frequency_penalty=-0.02),                   # pulled toward what it has seen most
        dict(logit_bias={prompt[0]: 0.3, prompt[1]: -0.3, 7: 0.25}),           # a bias and nothing else: no counts
        dict(),
        dict(temperature=0.8, top_k=40, seed=900 + i, repetition_penalty=1.2, frequency_penalty=0.01),
        dict(repetition_penalty=0.6, presence_penalty=0.01, logit_bias={prompt[2]: 0.2}),
    ]
    return SamplingParams(**kinds[i % len(kinds)], **common)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_with_penalties_under_preemption_matches_the_plain_implementation(tmp_path, dtype):
    from tandemllm_b200.engine import Engine, EngineArgs
    cfg = T.TINY_C
    W = random_model_weights(cfg, T.SEEDS["c"], T.STD["c"], bf16_exact=True)
    folder = write_folder(str(tmp_path / "c"), cfg, W, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    g = torch.Generator().manual_seed(23)
    n_req, new_tokens = 12, 28
    lengths = [int(torch.randint(12, 150, (1,), generator=g)) for _ in range(n_req)]
    prompts = []
    for n in lengths:                               # prompts over a few tokens each: the prompt's counts are above one
        few = torch.randint(0, cfg["vocab_size"], (max(3, n // 5),), generator=g)
        prompts.append(few[torch.randint(0, few.numel(), (n,), generator=g)].tolist())
    budget = -(-(max(lengths) + new_tokens + 40) // 16) * 16
    eng = Engine.from_folder(folder, EngineArgs(dtype=dtype, max_len=max(lengths) + new_tokens + 8, parallel=5, block_size=16,
                                                kv_blocks=budget // 16, max_batched_tokens=96, chunk_size=48))
    params = [_params(i, new_tokens, prompts[i]) for i in range(n_req)]
    outs = eng.generate(prompts, params)
    eng.cache.check()
    assert eng.scheduler.stats.preemptions > 0 and all(len(o) == new_tokens for o in outs)
    exact = total = moved = 0
    for i, (prompt, out, sp) in enumerate(zip(prompts, outs, params)):
        seq = list(prompt)
        for tok in out:
            raw = P.forward(cfg, W, seq)[-1]
            ref = P.penalize(raw, seq, sp.repetition_penalty, sp.presence_penalty, sp.frequency_penalty, sp.logit_bias)
            if sp.temperature == 0.0:
                best = int(ref.argmax())
                moved += best != int(raw.argmax())
                if tok != best:              # only where the precision cannot tell the two apart
                    assert float(ref[best] - ref[tok]) <= 2 * TOL[dtype] * float(raw.abs().max()), (i, len(seq), tok, best)
            else:
                best = P.sample(ref, sp.temperature, sp.top_k, sp.top_p, sp.min_p, seed=sp.seed, position=len(seq))
            exact += tok == best
            total += 1
            seq.append(tok)
    assert moved > total // 8, "the penalties changed the choice often enough for the comparison to mean something"
    if dtype == "float32":
        assert exact == total, (exact, total)
    else:
        assert exact >= int(0.9 * total), (exact, total)
    # the same requests alone, with room for everything, give the same tokens in 32-bit
    if dtype == "float32":
        roomy = Engine.from_folder(folder, EngineArgs(dtype=dtype, max_len=max(lengths) + new_tokens + 8, parallel=1,
                                                      block_size=16))
        for i in (0, 1, 4):
            assert roomy.generate([prompts[i]], [_params(i, new_tokens, prompts[i])])[0] == outs[i], i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_with_the_no_repeat_rule_and_the_pattern_stop_matches_the_plain_implementation(tmp_path, dtype):
    """`no_repeat_ngram_size` alone, beside a bias on one of the blocked tokens, beside the count penalties and under
    temperature; and a request that is ended by a repeating pattern. Every token is held to the plain implementation run on
    the text so far, with the rule's blocked set found by brute force; requests without the rule decode beside them (and a
    step is launched ahead only when no running request has the rule)."""
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    from tandemllm_b200.sampling.sampler import NO_REPEAT_PENALTY
    cfg = T.TINY_C
    W = random_model_weights(cfg, T.SEEDS["c"], T.STD["c"], bf16_exact=True)
    folder = write_folder(str(tmp_path / "c"), cfg, W, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    g = torch.Generator().manual_seed(31)
    new_tokens = 40
    prompts = []
    for n in (30, 90, 14, 55, 70, 21):              # prompts over a few tokens each: n-grams repeat inside the prompt already
        few = torch.randint(0, cfg["vocab_size"], (4,), generator=g)
        prompts.append(few[torch.randint(0, 4, (n,), generator=g)].tolist())
    common = dict(max_tokens=new_tokens, ignore_eos=True)
    params = [SamplingParams(no_repeat_ngram_size=2, **common),
              SamplingParams(no_repeat_ngram_size=3, logit_bias={prompts[1][0]: 1.0, prompts[1][1]: -0.5}, **common),
              SamplingParams(**common),
              SamplingParams(no_repeat_ngram_size=2, repetition_penalty=1.3, presence_penalty=0.2, **common),
              SamplingParams(no_repeat_ngram_size=4, temperature=0.7, top_k=30, seed=77, **common),
              SamplingParams(max_pattern_size=3, min_pattern_size=1, min_count=3, **common)]
    eng = Engine.from_folder(folder, EngineArgs(dtype=dtype, max_len=160, parallel=4, block_size=16, max_batched_tokens=64,
                                                chunk_size=32))
    reqs = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
    while eng.scheduler.has_unfinished():
        eng.run_step()
    outs = [r.output for r in reqs]
    assert all(len(o) == new_tokens for o in outs[:5])
    exact = total = blocked_moves = 0
    for i, (prompt, out, sp) in enumerate(zip(prompts, outs, params)):
        seq, calls = list(prompt), [list(prompt)]
        for k, tok in enumerate(out):
            raw = P.forward(cfg, W, seq)[-1]
            bias = dict(sp.logit_bias or {})
            if sp.no_repeat_ngram_size:
                for t in P.no_repeat_blocked(calls, sp.no_repeat_ngram_size):
                    bias[t] = bias.get(t, 0.0) - NO_REPEAT_PENALTY
            ref = P.penalize(raw, seq, sp.repetition_penalty, sp.presence_penalty, sp.frequency_penalty, bias)
            if sp.temperature == 0.0:
                best = int(ref.argmax())
                blocked_moves += bool(sp.no_repeat_ngram_size) and best != int(raw.argmax())
                if tok != best:
                    assert float(ref[best] - ref[tok]) <= 2 * TOL[dtype] * float(raw.abs().max()), (i, k, tok, best)
            else:
                best = P.sample(ref, sp.temperature, sp.top_k, sp.top_p, sp.min_p, seed=sp.seed, position=len(seq))
            exact += tok == best
            total += 1
            seq.append(tok)
            calls.append([tok])
            if sp.stops_on_patterns:
                ended = P.pattern_ends(out[:k + 1], sp.min_pattern_size, sp.max_pattern_size, sp.min_count)
                assert ended == (k == len(out) - 1 and reqs[i].finish_reason == "stop"), (i, k)
    assert blocked_moves > 10, "the rule changed the choice often enough for the comparison to mean something"
    if dtype == "float32":
        assert exact == total, (exact, total)
    else:
        assert exact >= int(0.9 * total), (exact, total)
    last = reqs[5]
    assert last.finish_reason in ("stop", "length") and (last.stop_pattern is not None) == (last.finish_reason == "stop")
    # greedy decoding of a tiny random model falls into a loop: the pattern stop must have seen it
    assert last.finish_reason == "stop" and len(last.output) < new_tokens
    assert 1 <= len(last.stop_pattern) <= 3 and last.output[-3 * len(last.stop_pattern):] == list(last.stop_pattern) * 3
