"""Configurations with sizes no kernel is tuned for (a head size of 48 and of 80, groups of 1 and 3, 2 and 5 conv taps,
top-1 and top-all routing, widths that are no multiple of 8, odd vocabularies), replayed the four ways against the
plain implementation in both precisions: every size the configuration allows is either computed right or refused
with an error, never computed wrongly."""

import pytest

from tests import plain_lfm2 as P
from tests import tiny_configs as T
from tests import traces
from tests.test_gpu_replay import LENGTHS, Case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=[("d", "float32"), ("d", "bfloat16"), ("e", "float32"), ("e", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def odd(request, tmp_path_factory):
    return Case(request.param[0], request.param[1], tmp_path_factory.mktemp("odd"))


def test_whole_decoded_tail_portions_and_mixed(odd):
    eng = odd.engine(max_tokens=256)
    odd.compare(odd.replay(eng, traces.whole(odd.requests)), "whole")
    odd.compare(odd.replay(eng, traces.decoded_tail(odd.requests, 32)), "decoded tail")
    odd.compare(odd.replay(eng, traces.portions(odd.requests)), "portions")
    trace = traces.mixed(odd.requests, live=4, seed=1)
    held = traces.tokens_held(trace, 64)
    assert held < sum(-(-n // 64) * 64 for n in LENGTHS)
    tight = odd.engine(max_tokens=held)
    odd.compare(odd.replay(tight, trace), "mixed on few pages")
    assert tight.cache.groups[0].pool.reused > 0


def test_greedy_generation(odd):
    from tandemllm_b200.sampling import SamplingParams
    from tests.test_gpu_replay import greedy_like_plain
    eng = odd.engine(max_tokens=512)
    prompts = [odd.requests["q2"][:20], odd.requests["q5"][:7]]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert len(out) == 10
        greedy_like_plain(odd, prompt, out)
