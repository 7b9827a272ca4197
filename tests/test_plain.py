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
