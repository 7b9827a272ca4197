"""The random-weights mode: a model from a configuration and a seed.

`write_model_folder` writes config.json and model.safetensors, so that everything downstream (loader,
engine, replay) reads a random model exactly as it reads a real one. `random_weights` yields the same
kind of tensors in memory, on any device, for sizes that should not pass through a file.

Every tensor is drawn from its own generator seeded by (seed, name), so a tensor's values do not depend
on which other tensors exist or on the order they are made in. Matrices are N(0, std), norm weights
1 + N(0, norm_std) (exactly 1 by default), biases N(0, bias_std). The reference has such a generator in
its tests only (tests/test_lfm2_moe_ref.py:39-74).
"""

from __future__ import annotations

import json
import os
import zlib
from typing import Iterable

import torch

from .loader import TensorSpec
from .safetensors_io import write_file


def _tensor_seed(seed: int, name: str) -> int:
    x = (int(seed) * 0x9E3779B97F4A7C15 + zlib.crc32(name.encode()) + 1) & ((1 << 64) - 1)
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & ((1 << 64) - 1)
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & ((1 << 64) - 1)
    return (x ^ (x >> 31)) >> 1


def random_tensor(spec: TensorSpec, seed: int, std: float, bias_std: float, norm_std: float,
                  device="cpu") -> torch.Tensor:
    """The 32-bit random tensor of `spec`."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32, device=device)
    t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
    if spec.init == "ones":
        return 1.0 + norm_std * t if norm_std else torch.ones(spec.shape, dtype=torch.float32, device=device)
    return t * (bias_std if spec.init == "bias" else std)


def random_weights(specs: Iterable[TensorSpec], seed: int, std: float = 0.02, bias_std: float = 0.1,
                   norm_std: float = 0.0, dtype: torch.dtype = torch.bfloat16, device="cpu") -> dict[str, torch.Tensor]:
    """name -> tensor: matrices in `dtype`, vectors in 32-bit."""
    out = {}
    for s in specs:
        t = random_tensor(s, seed, std, bias_std, norm_std, device)
        out[s.name] = t.to(dtype) if s.role == "matrix" else t
    return out


def write_model_folder(config, folder: str, seed: int, std: float = 0.02, bias_std: float = 0.1, norm_std: float = 0.0,
                       dtype: torch.dtype = torch.bfloat16, name_prefix: str = "model.") -> str:
    """Write `folder/config.json` and `folder/model.safetensors` for the typed `config` (anything with
    `to_dict()` and `to_spec()`), random weights from `seed`. Matrices are stored in `dtype`; vectors that the
    engine keeps in 32-bit (the expert bias) are stored in 32-bit when `dtype` is float32, else in `dtype`,
    except biases, which are always 32-bit."""
    from ..parts.model import DecoderModel      # the parts say which tensors a model reads
    os.makedirs(folder, exist_ok=True)
    spec = config.to_spec()
    model = DecoderModel(spec)
    tensors = {}
    for s in model.weight_specs(None):
        t = random_tensor(s, seed, std, bias_std, norm_std)
        keep32 = s.init == "bias" or dtype == torch.float32
        stored = s.name if s.name == spec.head_name else name_prefix + s.name
        tensors[stored] = t if keep32 else t.to(dtype)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_file(os.path.join(folder, "model.safetensors"), tensors,
               metadata={"format": "pt", "seed": str(seed), "std": str(std)})
    return folder
