"""The tiny LFM2 MoE configurations of the tests, as config.json dictionaries, and their prompts.

A and B differ in every size and option: layer count and order, width, head counts and grouping, head size,
conv taps and conv bias, dense layer count and width, expert count, top-k, expert width, expert bias,
renormalisation, scaling factor, vocabulary, rotary base, norm eps, tied or untied head. Widths and the
vocabulary of B are no powers of two.
"""

from __future__ import annotations

import torch

TINY_A = dict(
    model_type="lfm2_moe", architectures=["Lfm2MoeForCausalLM"], vocab_size=256, hidden_size=64,
    intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=4, num_attention_heads=4,
    num_key_value_heads=2, head_dim=16, norm_eps=1e-5, max_position_embeddings=4096, conv_bias=False,
    conv_L_cache=3, num_dense_layers=1, num_experts=4, num_experts_per_tok=2, use_expert_bias=True,
    routed_scaling_factor=1.0, norm_topk_prob=True, tie_word_embeddings=True,
    layer_types=["conv", "full_attention", "conv", "full_attention"],
    rope_parameters={"rope_type": "default", "rope_theta": 10000.0}, eos_token_id=2, bos_token_id=1, pad_token_id=0,
)

TINY_B = dict(
    model_type="lfm2_moe", architectures=["Lfm2MoeForCausalLM"], vocab_size=384, hidden_size=96,
    intermediate_size=256, moe_intermediate_size=48, num_hidden_layers=6, num_attention_heads=3,
    num_key_value_heads=1, head_dim=32, norm_eps=1e-6, max_position_embeddings=4096, conv_bias=True,
    conv_L_cache=4, num_dense_layers=2, num_experts=8, num_experts_per_tok=3, use_expert_bias=False,
    routed_scaling_factor=1.5, norm_topk_prob=False, tie_word_embeddings=False,
    layer_types=["conv", "conv", "full_attention", "conv", "full_attention", "full_attention"],
    rope_parameters={"rope_type": "default", "rope_theta": 1000000.0}, eos_token_id=3, bos_token_id=1, pad_token_id=0,
)

# A third model with the head size (64) and the widths (multiples of 8) that the tensor-core kernels of the bfloat16
# path take, so that the replay tests run those kernels too; it starts with an attention layer and ends with a conv.
TINY_C = dict(
    model_type="lfm2_moe", architectures=["Lfm2MoeForCausalLM"], vocab_size=320, hidden_size=128,
    intermediate_size=192, moe_intermediate_size=64, num_hidden_layers=4, num_attention_heads=4,
    num_key_value_heads=1, head_dim=64, norm_eps=1e-5, max_position_embeddings=4096, conv_bias=False,
    conv_L_cache=3, num_dense_layers=1, num_experts=6, num_experts_per_tok=2, use_expert_bias=True,
    routed_scaling_factor=1.0, norm_topk_prob=True, tie_word_embeddings=True,
    layer_types=["full_attention", "conv", "full_attention", "conv"],
    rope_parameters={"rope_type": "default", "rope_theta": 1000000.0}, eos_token_id=2, bos_token_id=1, pad_token_id=0,
)

# Two more with sizes no kernel is tuned for. D: a head size of 48 (a multiple of 16 that is no power of two), as many KV
# heads as query heads, two conv taps, top-1 of 5 experts, no dense layer, an odd vocabulary, attention first. E: a head
# size of 80, three query heads a KV head, five conv taps with bias, every expert chosen (top-7 of 7), an expert width that
# is no multiple of 8 (the tensor-core kernels cannot take it and must say so to their caller, not compute wrongly), a
# scaling factor, an untied head.
TINY_D = dict(
    model_type="lfm2_moe", architectures=["Lfm2MoeForCausalLM"], vocab_size=1001, hidden_size=80,
    intermediate_size=144, moe_intermediate_size=40, num_hidden_layers=3, num_attention_heads=5,
    num_key_value_heads=5, head_dim=48, norm_eps=1e-5, max_position_embeddings=4096, conv_bias=False,
    conv_L_cache=2, num_dense_layers=0, num_experts=5, num_experts_per_tok=1, use_expert_bias=True,
    routed_scaling_factor=1.0, norm_topk_prob=True, tie_word_embeddings=True,
    layer_types=["full_attention", "full_attention", "conv"],
    rope_parameters={"rope_type": "default", "rope_theta": 50000.0}, eos_token_id=2, bos_token_id=1, pad_token_id=0,
)

TINY_E = dict(
    model_type="lfm2_moe", architectures=["Lfm2MoeForCausalLM"], vocab_size=517, hidden_size=136,
    intermediate_size=100, moe_intermediate_size=28, num_hidden_layers=5, num_attention_heads=6,
    num_key_value_heads=2, head_dim=80, norm_eps=3e-6, max_position_embeddings=4096, conv_bias=True,
    conv_L_cache=5, num_dense_layers=1, num_experts=7, num_experts_per_tok=7, use_expert_bias=False,
    routed_scaling_factor=0.7, norm_topk_prob=False, tie_word_embeddings=False,
    layer_types=["conv", "full_attention", "conv", "conv", "full_attention"],
    rope_parameters={"rope_type": "default", "rope_theta": 1000000.0}, eos_token_id=2, bos_token_id=1, pad_token_id=0,
)

# B without the three options the reference refuses, so the reference itself can run it
TINY_B_REFERENCE = {**TINY_B, "conv_bias": False, "norm_topk_prob": True}

SEEDS = {"a": 0, "b": 1, "c": 2, "d": 3, "e": 4}
STD = {"a": 0.02, "b": 0.05, "c": 0.02, "d": 0.04, "e": 0.03}
CONFIGS = {"a": TINY_A, "b": TINY_B, "c": TINY_C, "d": TINY_D, "e": TINY_E}


def prompts(name: str) -> list[list[int]]:
    """Seeded uniform-random token ids: A has prompts of 16 and 9 tokens, B of 33, 5 and 20, C of 70 and 12."""
    lens, seed = {"a": ((16, 9), 100), "b": ((33, 5, 20), 101), "c": ((70, 12), 102)}[name]
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, CONFIGS[name]["vocab_size"], (n,), generator=g).tolist() for n in lens]


def long_tokens(name: str, n: int, seed: int = 7) -> list[int]:
    cfg = CONFIGS[name]
    g = torch.Generator().manual_seed(seed * 1000 + n)
    return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
