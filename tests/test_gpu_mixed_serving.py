"""Mixed serving through the scheduler, held to the plain implementation: a dozen requests whose prompts are log-uniform in
length, fed as portions beside the decode rows of others, on a cache budget so small that requests queue, pages are used
again and running requests are preempted and recomputed; greedy and seeded temperature sampling alternate. Every generated
token is checked against the plain implementation run on the text so far (teacher-forced): the measurement program's
scenario (`bench.py --scenario mixed`) at a size where that is affordable."""

import math

import pytest
import torch

from tests import plain_lfm2 as P
from tests import tiny_configs as T
from tests.helpers import random_model_weights, write_folder

pytestmark = pytest.mark.gpu
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_serving_under_a_tight_cache_budget_matches_the_plain_implementation(tmp_path, dtype):
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    cfg = T.TINY_C
    W = random_model_weights(cfg, T.SEEDS["c"], T.STD["c"], bf16_exact=True)
    folder = write_folder(str(tmp_path / "c"), cfg, W, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    g = torch.Generator().manual_seed(11)
    n_req, new_tokens = 12, 36
    lengths = [int(math.exp(math.log(16) + float(torch.rand(1, generator=g)) * math.log(400 / 16))) for _ in range(n_req)]
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
    budget = -(-(max(lengths) + new_tokens + 40) // 16) * 16      # the longest request and little more: never all twelve
    assert budget < sum(lengths) // 2
    eng = Engine.from_folder(folder, EngineArgs(dtype=dtype, max_len=max(lengths) + new_tokens + 8, parallel=6, block_size=16,
                                                kv_blocks=budget // 16, max_batched_tokens=160, chunk_size=64,
                                                record_routing=True))
    params = [SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True) if i % 2 == 0 else
              SamplingParams(temperature=0.8, top_k=50, top_p=0.95, seed=100 + i, max_tokens=new_tokens, ignore_eos=True)
              for i in range(n_req)]
    outs = eng.generate(prompts, params)
    st = eng.scheduler.stats
    eng.cache.check()
    assert all(len(o) == new_tokens for o in outs)
    assert st.preemptions > 0 and eng.cache.groups[0].pool.reused > 0 and st.prompt_rows > sum(lengths)   # recomputed text
    mixed_steps = [r for r in eng.records if r["decode_rows"] and r["prompt_rows"]]
    assert mixed_steps, "portions ran beside decode rows"
    assert all(r["pages_used"][0] <= budget // 16 for r in eng.records)
    exact = agree = total = 0
    for i, (prompt, out, sp) in enumerate(zip(prompts, outs, params)):
        seq = list(prompt)
        for tok in out:
            ref = P.forward(cfg, W, seq)[-1]
            if sp.temperature == 0.0:
                best = int(ref.argmax())
                if tok != best:              # only where the precision cannot tell the two apart
                    assert float(ref[best] - ref[tok]) <= 2 * TOL[dtype] * float(ref.abs().max()), (i, len(seq), tok, best)
                exact += tok == best
            else:
                agree += tok == P.sample(ref, 0.8, 50, 0.95, 0.0, seed=sp.seed, position=len(seq))
            total += 1
            seq.append(tok)
    half = total // 2
    if dtype == "float32":
        assert exact == half and agree == half, (exact, agree, half)
    else:
        assert exact >= int(0.9 * half) and agree >= int(0.8 * half), (exact, agree, half)
