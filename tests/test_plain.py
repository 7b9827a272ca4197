"""The plain implementation against the reference's own model code (numbers stored by
tests/golden/make_golden.py), and its parts against each other."""

import os

import numpy as np
import pytest
import torch

from tests import plain_lfm2 as P
from tests import tiny_configs as T
from tests.helpers import random_model_weights

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _checksum(W):
    return float(sum(float(t.double().abs().sum()) for _, t in sorted(W.items())))


@pytest.mark.parametrize("name,cfg", [("a", T.TINY_A), ("b", T.TINY_B_REFERENCE)])
def test_plain_matches_reference_logits(name, cfg):
    g = np.load(os.path.join(GOLDEN, f"tiny_{name}_reference.npz"))
    W = random_model_weights(cfg, T.SEEDS[name], T.STD[name])
    assert abs(_checksum(W) - float(g["weights_checksum"])) < 1e-6 * float(g["weights_checksum"]), \
        "the seeded weights changed; run tests/golden/make_golden.py again"
    for i, prompt in enumerate(T.prompts(name)):
        assert prompt == g[f"prompt_{i}"].tolist()
        ref = torch.from_numpy(g[f"logits_{i}"])
        got = P.forward(cfg, W, prompt)
        assert float((got - ref).abs().max()) < 2e-5, f"model {name} prompt {i}"


def test_causality_a_prefix_gives_the_same_logits():
    W = random_model_weights(T.TINY_B, 1, 0.05)
    toks = T.long_tokens("b", 40)
    whole = P.forward(T.TINY_B, W, toks)
    part = P.forward(T.TINY_B, W, toks[:23])
    assert float((whole[:23] - part).abs().max()) < 1e-5


def test_options_change_the_result():
    """Each option the reference pins moves the logits, so a test that ignores it would fail."""
    W = random_model_weights(T.TINY_B, 1, 0.05)
    toks = T.long_tokens("b", 12)
    base = P.forward(T.TINY_B, W, toks)
    for key, other in (("conv_bias", False), ("norm_topk_prob", True), ("routed_scaling_factor", 1.0)):
        moved = P.forward({**T.TINY_B, key: other}, W, toks)
        assert float((moved - base).abs().max()) > 1e-4, key
    tied = P.forward({**T.TINY_B, "tie_word_embeddings": True}, W, toks)
    assert float((tied - base).abs().max()) > 1e-4


def test_router_ties_go_to_the_lower_id():
    cfg = {**T.TINY_A, "use_expert_bias": False}
    W = {"gate.weight": torch.zeros(4, 64)}
    ids, w = P.route(torch.randn(3, 64), W, "", cfg)
    assert ids.tolist() == [[0, 1]] * 3
    assert torch.allclose(w, torch.full((3, 2), 0.5 / (1.0 + 1e-6)))


def test_sampling_filters_and_keyed_draws():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(200, generator=g) * 3
    keep = P.kept_tokens(logits, 0.7, top_k=10, top_p=1.0, min_p=0.0)
    assert int(keep.sum()) == 10 and bool(keep[logits.argmax()])
    keep = P.kept_tokens(logits, 0.7, top_k=0, top_p=0.5, min_p=0.0)
    p = torch.softmax(logits.double() / 0.7, -1)
    assert float(p[keep].sum()) >= 0.5 and float(p[keep].sum() - p[keep].min()) <= 0.5 + 1e-12
    keep = P.kept_tokens(logits, 1.0, top_k=0, top_p=1.0, min_p=0.2)
    assert bool((p.new_tensor(1.0) * torch.softmax(logits.double(), -1)[keep] >= 0.2 * torch.softmax(logits.double(), -1).max() - 1e-12).all())
    a = P.sample(logits, 0.7, 20, 0.9, 0.0, seed=11, position=5)
    assert a == P.sample(logits, 0.7, 20, 0.9, 0.0, seed=11, position=5)
    draws = {P.sample(logits, 1.5, 0, 1.0, 0.0, seed=s, position=5) for s in range(40)}
    assert len(draws) > 5
    assert P.sample(logits, 0.0, 5, 0.5, 0.1, seed=1, position=0) == int(logits.argmax())
    assert 0.0 < P.keyed_uniform(1, 2, 3) < 1.0


def test_penalties_on_a_hand_made_row():
    logits = torch.tensor([2.0, -2.0, 1.0, -1.0, 0.5, 3.0])
    history = [0, 1, 1, 5, 5, 5]
    out = P.penalize(logits, history, repetition=2.0)
    assert out.tolist() == [1.0, -4.0, 1.0, -1.0, 0.5, 1.5]           # seen and positive: halved; seen and negative: doubled
    out = P.penalize(logits, history, presence=0.5, frequency=0.25)
    assert out.tolist() == [2.0 - 0.5 - 0.25, -2.0 - 0.5 - 0.5, 1.0, -1.0, 0.5, 3.0 - 0.5 - 0.75]
    # the bias comes first: token 2 is unseen, so only the bias moves it; token 1 turns positive before the repetition rule
    out = P.penalize(logits, history, repetition=2.0, bias={1: 3.0, 2: -4.0})
    assert out.tolist() == [1.0, 0.5, -3.0, -1.0, 0.5, 1.5]
    assert torch.equal(P.penalize(logits, history), logits)


def test_the_no_repeat_index_equals_the_brute_force_rule_across_the_window():
    """`NoRepeatIndex` (the product's memory of the rule) against `plain_lfm2.no_repeat_blocked` (no index, the kept text
    searched each time), over prompts shorter and longer than the window, so that the forgetting of the older half is
    crossed once by the prompt and again token by token."""
    import random

    from tandemllm_b200.sampling import NoRepeatIndex
    rnd = random.Random(3)
    for n in (2, 3, 5):
        for prompt_len, vocab, steps in ((0, 3, 40), (7, 4, 60), (1500, 6, 700), (2100, 5, 30), (5000, 50, 1200)):
            prompt = [rnd.randrange(vocab) for _ in range(prompt_len)]
            index, calls = NoRepeatIndex(n), [prompt]
            index.add(prompt)
            for step in range(steps):
                assert index.blocked() == P.no_repeat_blocked(calls, n), (n, prompt_len, step)
                t = rnd.randrange(vocab)
                index.add([t])
                calls.append([t])
            assert index.seen == prompt_len + steps


def test_the_pattern_stop_equals_the_plain_rule_and_the_parameters_are_checked():
    import random

    from tandemllm_b200.sampling import SamplingParams, repeating_pattern
    rnd = random.Random(4)
    hits = 0
    for _ in range(3000):
        toks = [rnd.randrange(3) for _ in range(rnd.randrange(0, 30))]
        lo = rnd.randrange(1, 4)
        hi, count = rnd.randrange(lo, 6), rnd.randrange(2, 5)
        got = repeating_pattern(toks, lo, hi, count)
        assert (got is not None) == P.pattern_ends(toks, lo, hi, count)
        if got is not None:
            hits += 1
            assert lo <= len(got) <= hi and toks[-len(got) * count:] == list(got) * count
    assert hits > 100
    assert repeating_pattern([5, 5, 5, 5], 1, 2, 4) == (5,) and repeating_pattern([1, 2, 1, 2], 1, 2, 2) == (1, 2)
    assert not SamplingParams().stops_on_patterns and not SamplingParams(max_pattern_size=4, min_count=1).stops_on_patterns
    assert SamplingParams(max_pattern_size=4, min_count=2).stops_on_patterns
    assert SamplingParams(no_repeat_ngram_size=3).changes_logits and not SamplingParams(no_repeat_ngram_size=3).penalizes
    for bad in (dict(no_repeat_ngram_size=1), dict(no_repeat_ngram_size=-2), dict(min_pattern_size=0), dict(max_pattern_size=-1)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


def test_the_filters_of_a_sampled_request_come_from_the_request_the_flags_the_card_or_nowhere(tmp_path):
    """`sampling.defaults.resolve` (the reference's server/sampling_defaults.py:41-66): the first of request, flags and
    card that names a filter decides all three; what the request leaves out comes from the flags, never from the card."""
    import json

    from tandemllm_b200.sampling import card_sampling, resolve_filters
    card = {"top_p": 0.95, "top_k": 20}
    assert resolve_filters({}, None, None) == {"top_p": 1.0, "top_k": 0, "min_p": 0.0, "source": "none"}
    assert resolve_filters({"temperature": 0.7}, None, card) == {"top_p": 0.95, "top_k": 20, "min_p": 0.0, "source": "card"}
    assert resolve_filters({"top_k": None}, {"top_p": 0.8}, card) == {"top_p": 0.8, "top_k": 0, "min_p": 0.0, "source": "flags"}
    assert resolve_filters({"min_p": 0.1}, {"top_p": 0.8, "top_k": None}, card) == \
        {"top_p": 0.8, "top_k": 0, "min_p": 0.1, "source": "request"}
    assert resolve_filters({"top_k": "40"}, None, card) == {"top_p": 1.0, "top_k": 40, "min_p": 0.0, "source": "request"}
    assert resolve_filters(None, None, {"top_k": None, "top_p": 0.9})["top_k"] == 0
    with pytest.raises(ValueError):
        resolve_filters({"top_p": "much"})
    assert card_sampling(str(tmp_path)) is None
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 7, "top_k": 50, "temperature": 0.1}))
    assert card_sampling(str(tmp_path)) == {"top_k": 50}
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 7}))
    assert card_sampling(str(tmp_path)) is None
