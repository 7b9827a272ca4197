"""Randomly drawn configurations of the architecture (every size and option within what config.json allows), each replayed
whole and mixed with few pages against the plain implementation in both precisions. The draws are seeded, so a failure
names its configuration; what a kernel does not take it must refuse with an error that says so, never compute wrongly."""

import random

import pytest

from tests import tiny_configs as T
from tests import traces
from tests.test_gpu_replay import Case

pytestmark = pytest.mark.gpu


def draw(seed: int) -> dict:
    rng = random.Random(seed)
    head_dim = rng.choice([16, 32, 48, 64, 64, 80, 96, 128, 256])
    kv = rng.choice([1, 1, 2, 3, 4])
    group = rng.choice([1, 2, 3, 4, 7])
    layers = rng.randint(2, 5)
    kinds = [rng.choice(["conv", "full_attention"]) for _ in range(layers)]
    if "full_attention" not in kinds:
        kinds[rng.randrange(layers)] = "full_attention"
    experts = rng.choice([1, 2, 3, 5, 8, 9, 33, 40, 70])
    return dict(
        model_type="lfm2_moe", architectures=["Lfm2MoeForCausalLM"], vocab_size=rng.choice([97, 250, 511, 1030, 3001]),
        hidden_size=rng.choice([48, 72, 90, 100, 136, 200, 264]), intermediate_size=rng.choice([40, 64, 100, 136, 250]),
        moe_intermediate_size=rng.choice([8, 24, 28, 40, 64]), num_hidden_layers=layers, num_attention_heads=kv * group,
        num_key_value_heads=kv, head_dim=head_dim, norm_eps=rng.choice([1e-5, 1e-6, 3e-6]), max_position_embeddings=4096,
        conv_bias=rng.random() < 0.4, conv_L_cache=rng.choice([2, 3, 3, 4, 6]), num_dense_layers=rng.randint(0, layers - 1),
        num_experts=experts, num_experts_per_tok=rng.randint(1, min(experts, 8)), use_expert_bias=rng.random() < 0.6,
        routed_scaling_factor=rng.choice([1.0, 1.0, 0.5, 2.5]), norm_topk_prob=rng.random() < 0.7,
        tie_word_embeddings=rng.random() < 0.6, layer_types=kinds,
        rope_parameters={"rope_type": "default", "rope_theta": rng.choice([1e4, 5e5, 1e6])}, eos_token_id=2, bos_token_id=1,
        pad_token_id=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(1, 17)))
def test_a_drawn_configuration_replays_like_the_plain_implementation(seed, dtype, tmp_path_factory):
    from tandemllm_b200.kernels.ops import KernelError
    name = f"fuzz{seed}"
    T.CONFIGS[name], T.SEEDS[name], T.STD[name] = draw(seed), 100 + seed, 0.04
    try:
        case = Case(name, dtype, tmp_path_factory.mktemp(name))
        try:
            eng = case.engine(max_tokens=256)
            case.compare(case.replay(eng, traces.whole(case.requests)), f"whole {T.CONFIGS[name]}")
            trace = traces.mixed(case.requests, live=4, seed=seed)
            tight = case.engine(max_tokens=traces.tokens_held(trace, 64))
            case.compare(case.replay(tight, trace), f"mixed {T.CONFIGS[name]}")
        except (KernelError, ValueError) as refusal:
            # a size this engine does not take must be named in the refusal
            text = str(refusal)
            assert any(w in text for w in ("implemented", "multiple", "size", "taps", "experts", "head")), text
            pytest.skip(f"refused: {text[:200]}")
    finally:
        for d in (T.CONFIGS, T.SEEDS, T.STD):
            d.pop(name, None)
