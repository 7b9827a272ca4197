"""Shared helpers of the tests: random weights of a tiny configuration, model folders, comparisons."""

from __future__ import annotations

import json
import os

import torch

from tandemllm_b200.config import Lfm2MoeConfig
from tandemllm_b200.parts.model import DecoderModel
from tandemllm_b200.weights.random_init import random_tensor
from tandemllm_b200.weights.safetensors_io import write_file


def random_model_weights(cfg: dict, seed: int, std: float, norm_std: float = 0.1, bias_std: float = 0.1,
                         bf16_exact: bool = False) -> dict[str, torch.Tensor]:
    """32-bit weights by canonical name for the config.json dict `cfg`. Norm weights are 1 + N(0, norm_std) so
    that a dropped norm weight shows. With `bf16_exact` every value is rounded to a bfloat16 value."""
    config = Lfm2MoeConfig.from_dict(cfg)
    W = {}
    for s in DecoderModel(config.to_spec()).weight_specs(None):
        t = random_tensor(s, seed, std, bias_std, norm_std)
        W[s.name] = t.to(torch.bfloat16).float() if bf16_exact else t
    return W


def write_folder(folder: str, cfg: dict, W: dict[str, torch.Tensor], dtype=torch.float32, prefix: str = "model.") -> str:
    """A model folder (config.json, model.safetensors) holding W; floating tensors are stored in `dtype`,
    the expert bias always in 32-bit."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    stored = {}
    for name, t in W.items():
        key = name if name == "lm_head.weight" else prefix + name
        stored[key] = t if name.endswith("expert_bias") or not t.is_floating_point() else t.to(dtype)
    write_file(os.path.join(folder, "model.safetensors"), stored)
    return folder


def max_rel(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a - b| over the largest |b| of each row."""
    a, b = a.double(), b.double()
    scale = b.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((a - b).abs() / scale).max())
