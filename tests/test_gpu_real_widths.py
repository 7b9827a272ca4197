"""Both precisions at the layer sizes the benchmark runs, a few layers deep, against the plain implementation: the shapes
at which the kernels choose their forms (the persistent kernel above 128 rows, the swapped one below, the register-only
product for a few rows, the grouped products with and without fetched rows and split down projections, the router for 32
and 64 experts, the head over a vocabulary of 65536) are otherwise only tested kernel by kernel.

`test_the_benchmarks_layer_sizes...` has the real widths of the 8B-A1B and of the 24B-A2B-class configurations with three
layers (a short-conv layer with the dense feed-forward, an attention layer and a short-conv layer with routed experts:
fewer layers are no smaller layers). Its steps: a prompt of 2048 rows; portions of 512 beside prompts of a few tokens and
beside decode rows; decode steps of 64, 33, 17, 8 and 1 rows, each shape twice, so that with graphs on the second one is a
replay."""

import pytest
import torch

from tests import plain_lfm2 as P
from tests.helpers import random_model_weights

pytestmark = pytest.mark.gpu

WIDTHS = dict(
    model_type="lfm2_moe", architectures=["Lfm2MoeForCausalLM"], vocab_size=2048, hidden_size=2048,
    intermediate_size=7168, moe_intermediate_size=1792, num_hidden_layers=2, num_attention_heads=32,
    num_key_value_heads=8, head_dim=64, norm_eps=1e-5, max_position_embeddings=4096, conv_bias=False,
    conv_L_cache=3, num_dense_layers=1, num_experts=16, num_experts_per_tok=4, use_expert_bias=True,
    routed_scaling_factor=1.0, norm_topk_prob=True, tie_word_embeddings=True, layer_types=["conv", "full_attention"],
    rope_parameters={"rope_type": "default", "rope_theta": 1000000.0}, eos_token_id=2, bos_token_id=1, pad_token_id=0,
)


@pytest.mark.parametrize("heads,kv_heads,head_dim,product", [(32, 8, 64, "pair"), (16, 4, 128, "pair"), (32, 8, 64, "single")])
def test_two_layers_at_the_benchmark_widths_against_the_plain_implementation(heads, kv_heads, head_dim, product, monkeypatch):
    """(`product`: the prompt-sized products on pairs of SMs, the default, or through the one-CTA kernel kept beside it)"""
    from tandemllm_b200.kernels import tensorcore
    monkeypatch.setattr(tensorcore, "PROMPT_PRODUCT", product)
    from tandemllm_b200.config import Lfm2MoeConfig
    from tandemllm_b200.engine import Engine, EngineArgs, StepEntry
    from tandemllm_b200.weights.loader import DictWeights
    WIDE = {**WIDTHS, "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim}
    W = random_model_weights(WIDE, 4, 0.02, bf16_exact=True)
    g = torch.Generator().manual_seed(9)
    seqs = {"p": torch.randint(0, 2048, (190,), generator=g).tolist(), "q": torch.randint(0, 2048, (60,), generator=g).tolist()}
    ref, margin = {}, {}
    for rid, toks in seqs.items():
        margins = []
        ref[rid] = P.forward(WIDE, W, toks, margins=margins)
        margin[rid] = torch.stack(margins).min(0).values
    spec = Lfm2MoeConfig.from_dict(WIDE).to_spec()
    for graph in (False, True):
        eng = Engine._build(None, spec, DictWeights({k: v.to(torch.bfloat16) if v.is_floating_point() and not k.endswith("expert_bias") else v
                                                     for k, v in W.items()}),
                            EngineArgs(dtype="bfloat16", max_len=512, parallel=2, graph=graph))
        eng.admit("p"), eng.admit("q")
        at = {"p": 0, "q": 0}
        got = {}

        def step(parts):
            entries = [StepEntry(r, seqs[r][at[r]:at[r] + n], list(range(n))) for r, n in parts]
            rows = eng.step(entries).float().cpu()
            k = 0
            for r, n in parts:
                for i in range(n):
                    got[(r, at[r] + i)] = rows[k]
                    k += 1
                at[r] += n
        step([("p", 140)])                         # more than 128 rows: the persistent kernels
        step([("p", 20), ("q", 40)])               # 60 rows: the swapped tcgen05 kernels, two requests
        step([("p", 10)])                          # a few rows: the register-only product, fetched expert rows
        while at["p"] < 190:                       # decoding, the two together while q lasts
            step([("p", 1)] + ([("q", 1)] if at["q"] < 60 else []))
        assert len(got) == 250
        bad, rerouted = [], 0
        for (r, pos), row in got.items():
            want = ref[r][pos]
            err = float((row - want).abs().max() / want.abs().max())
            if err > 3e-2:
                if float(margin[r][pos]) < 3e-2:
                    rerouted += 1                  # a routing near tie went the other way
                else:
                    bad.append((r, pos, round(err, 4), float(margin[r][pos])))
        assert not bad, f"graphs {graph}: {bad[:5]}"
        assert rerouted <= 25, rerouted


SIZES = {
    "8b": dict(intermediate_size=7168, moe_intermediate_size=1792, num_experts=32),
    "24b": dict(intermediate_size=11776, moe_intermediate_size=1536, num_experts=64),
}


class RealWidths:
    """Weights, token sequences and the plain implementation's logits for one of the benchmark's layer sizes (made once
    a size, used by both precisions: the weights are bfloat16 values, so the 32-bit engine and the plain implementation
    compute with the same numbers)."""
    _made: dict = {}

    def __init__(self, size: str):
        self.cfg = {**WIDTHS, **SIZES[size], "vocab_size": 65536, "num_hidden_layers": 3,
                    "layer_types": ["conv", "full_attention", "conv"], "num_dense_layers": 1, "max_position_embeddings": 8192}
        self.W = random_model_weights(self.cfg, 11, 0.02, bf16_exact=True)
        g = torch.Generator().manual_seed(21)
        V = self.cfg["vocab_size"]
        draw = lambda n: torch.randint(0, V, (n,), generator=g).tolist()
        self.seqs = {"p": draw(2048 + 3), "r": draw(1100)}
        self.seqs.update({f"d{i}": draw(4 + 2 * sum(i < n for n in (64, 33, 17, 8))) for i in range(64)})
        # the steps: (request, tokens fed, wanted places among them)
        at = {r: 0 for r in self.seqs}

        def take(r, n, want):
            e = (r, at[r], n, want)
            at[r] += n
            return e
        self.steps = [[take("p", 2048, [0, 1, 127, 128, 1000, 2046, 2047])]]
        self.steps.append([take("r", 512, [0, 300, 511])] + [take(f"d{i}", 3 if i < 8 else 4, [2]) for i in range(64)])
        self.steps.append([take("r", 512, [0, 511])] + [take(f"d{i}", 1, [0]) for i in range(8)])
        self.steps.append([take("r", 76, [0, 75])])
        for n in (64, 33, 17, 8):
            for _ in range(2):
                self.steps.append([take(f"d{i}", 1, [0]) for i in range(n)])
        for _ in range(3):
            self.steps.append([take("p", 1, [0])])
        assert all(at[r] == len(t) for r, t in self.seqs.items()), {r: (at[r], len(self.seqs[r])) for r in at if at[r] != len(self.seqs[r])}
        wanted = {}
        for step in self.steps:
            for r, start, n, want in step:
                wanted.setdefault(r, []).extend(start + w for w in want)
        self.ref, self.margin = {}, {}
        for r, toks in self.seqs.items():
            margins = []
            rows = sorted(set(wanted[r]))
            out = P.forward(self.cfg, self.W, toks, margins=margins, rows=rows)
            tight = torch.stack(margins).min(0).values
            for j, pos in enumerate(rows):
                self.ref[(r, pos)] = out[j]
                self.margin[(r, pos)] = float(tight[pos])

    @classmethod
    def get(cls, size: str) -> "RealWidths":
        if size not in cls._made:
            cls._made.clear()               # one size's weights at a time (a few GB of host memory each)
            cls._made[size] = cls(size)
        return cls._made[size]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", ["8b", "24b"])
def test_the_benchmarks_layer_sizes_against_the_plain_implementation(size, dtype):
    from tandemllm_b200.config import Lfm2MoeConfig
    from tandemllm_b200.engine import Engine, EngineArgs, StepEntry
    from tandemllm_b200.weights.loader import DictWeights
    case = RealWidths.get(size)
    spec = Lfm2MoeConfig.from_dict(case.cfg).to_spec()
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    weights = DictWeights({k: v.to(tdt) if v.is_floating_point() and not k.endswith("expert_bias") else v
                           for k, v in case.W.items()})
    eng = Engine._build(None, spec, weights, EngineArgs(dtype=dtype, max_len=4096, parallel=66, kv_blocks=400, graph=True))
    del weights
    got = {}
    for step in case.steps:
        entries = []
        for r, start, n, want in step:
            if not eng.cache.has(r):
                eng.admit(r)
            entries.append(StepEntry(r, case.seqs[r][start:start + n], want))
        rows = eng.step(entries).float().cpu()
        k = 0
        for r, start, n, want in step:
            for w in want:
                got[(r, start + w)] = rows[k]
                k += 1
        assert k == rows.shape[0]
    assert eng.step_function.graph_replays >= 5          # the second step of each decode shape came from its graph
    assert got.keys() == case.ref.keys()
    tol, near = (1e-4, 1e-5) if dtype == "float32" else (3e-2, 3e-2)
    bad, rerouted, worst = [], 0, 0.0
    for key, row in sorted(got.items()):
        want = case.ref[key]
        err = float((row - want).abs().max() / want.abs().max())
        if err <= tol:
            worst = max(worst, err)
        elif case.margin[key] < near:
            rerouted += 1                  # a routing near tie went the other way
        else:
            bad.append((key, round(err, 5), case.margin[key]))
    print(f"{size} {dtype}: {len(got)} positions, worst error {worst:.3g}, {rerouted} set aside as routing near ties")
    assert not bad, f"{size} {dtype}: {bad[:6]}"
    assert rerouted <= len(got) // 4, (rerouted, len(got))
    eng.cache.check()
