"""Mixed traces with contexts of more than a thousand tokens and up to eight live requests, at the head size and widths
the bfloat16 path's tensor-core kernels take (model C) and at model B's odd sizes: prompt portions on the tcgen05
attention beside decode rows on the small-tile form over shared key spans, pages of 16 to 128 tokens, few pages."""

import pytest
import torch

from tests import plain_lfm2 as P
from tests import tiny_configs as T
from tests import traces
from tests.test_gpu_replay import Case

pytestmark = pytest.mark.gpu
LONG = (1300, 40, 700, 260, 1100, 90, 513, 128, 64, 300)


@pytest.fixture(scope="module", params=[("c", "float32"), ("c", "bfloat16"), ("b", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def long_case(request, tmp_path_factory):
    case = Case(request.param[0], request.param[1], tmp_path_factory.mktemp("long"))
    case.requests = {f"L{i}": T.long_tokens(case.name, n, seed=60 + i) for i, n in enumerate(LONG)}
    case.ref, case.margin = {}, {}
    for rid, toks in case.requests.items():
        margins = []
        case.ref[rid] = P.forward(case.cfg, case.W, toks, margins=margins)
        case.margin[rid] = torch.stack(margins).min(0).values
    return case


@pytest.mark.parametrize("page,live,seed", [(16, 8, 0), (64, 5, 1), (128, 3, 2)])
def test_long_requests_mixed_on_few_pages(long_case, page, live, seed):
    trace = traces.mixed(long_case.requests, live=live, seed=seed, decode_after=0.9)
    held = -(-traces.tokens_held(trace, 64) // page) * page + live * page
    eng = long_case.engine(max_tokens=held, parallel=live, block_size=page)
    got = long_case.replay(eng, trace)
    assert len(got) == sum(LONG)
    long_case.compare(got, f"long mixed (pages of {page}, {live} live)")
    assert eng.cache.groups[0].pool.reused > 0
