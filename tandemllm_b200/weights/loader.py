"""Weights bound by tensor name.

A model's parts say which tensors they read (`TensorSpec`: name, shape, role); the loader checks a
folder's stored tensors against that list and raises ONE error that lists every missing tensor,
every unexpected one and every wrong shape, by name (the reference audits the same way before it
reads any data, engine/models/lfm2_moe/pack.py:205-252). Stored names may carry a prefix such as
`model.` (pack.py:59-60).

What is kept: floating tensors in bfloat16, except that a tensor stored in 32-bit stays 32-bit;
integer tables as int32. The model then casts matrices to its compute dtype and keeps vectors
(norm weights, biases, conv taps, the expert bias) in 32-bit.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Iterable

import torch

from .safetensors_io import CheckpointError, StoredTensor, index_folder, read_tensor


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part reads.

    role   "matrix" (multiplied; cast to the compute dtype), "vector" (kept in 32-bit) or "table"
           (integers, int32)
    init   how the random-weights mode fills it: "normal" (N(0, std)), "ones" (1 + N(0, norm_std)),
           "bias" (N(0, bias_std)) or "zeros"
    """
    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


def canonical_names(stored: Iterable[str], prefixes: tuple[str, ...]) -> dict[str, str]:
    """canonical name -> stored key, with one leading prefix stripped where present."""
    out: dict[str, str] = {}
    for key in stored:
        name = key
        for p in prefixes:
            if p and key.startswith(p):
                name = key[len(p):]
                break
        if name in out:
            raise CheckpointError(f"tensor {name} is stored twice: as {out[name]} and as {key}")
        out[name] = key
    return out


def kept_dtype(tag: str) -> torch.dtype:
    if tag in ("F32", "F64"):
        return torch.float32
    if tag in ("BF16", "F16"):
        return torch.bfloat16
    return torch.int32


def audit(expected: list[TensorSpec], stored: dict[str, StoredTensor], names: dict[str, str],
          where: str, ignore: Callable[[str], bool] | None = None) -> None:
    """Raise one CheckpointError listing missing and unexpected tensors and wrong shapes."""
    want = {s.name: s for s in expected}
    missing = sorted(n for n in want if n not in names)
    unexpected = sorted(n for n in names if n not in want and not (ignore and ignore(n)))
    wrong = []
    for n, s in want.items():
        if n in names:
            got = stored[names[n]].shape
            if tuple(got) != tuple(s.shape):
                wrong.append(f"{n}: stored {list(got)}, the configuration needs {list(s.shape)}")
    if missing or unexpected or wrong:
        def some(xs):
            return ", ".join(xs[:12]) + (f" and {len(xs) - 12} more" if len(xs) > 12 else "")
        parts = []
        if missing:
            parts.append(f"missing ({len(missing)}): {some(missing)}")
        if unexpected:
            parts.append(f"unexpected ({len(unexpected)}): {some(unexpected)}")
        if wrong:
            parts.append(f"wrong shape ({len(wrong)}): {some(sorted(wrong))}")
        raise CheckpointError(f"{where}: the stored tensors do not fit the configuration; " + "; ".join(parts))


class FolderWeights:
    """The stored tensors of a model folder, by canonical name."""

    def __init__(self, folder: str, prefixes: tuple[str, ...] = ("model.",)):
        self.folder = folder
        self.stored = index_folder(folder)
        self.names = canonical_names(self.stored, prefixes)

    def present(self) -> set[str]:
        return set(self.names)

    def check(self, expected: list[TensorSpec], ignore: Callable[[str], bool] | None = None) -> None:
        audit(expected, self.stored, self.names, self.folder, ignore)

    def read(self, name: str) -> torch.Tensor:
        st = self.stored[self.names[name]]
        t = read_tensor(st)
        return t.to(kept_dtype(st.dtype))


class DictWeights:
    """Tensors already in memory (the random-weights mode without a folder), same interface."""

    def __init__(self, tensors: dict[str, torch.Tensor]):
        self.tensors = tensors

    def present(self) -> set[str]:
        return set(self.tensors)

    def check(self, expected: list[TensorSpec], ignore: Callable[[str], bool] | None = None) -> None:
        stored = {n: StoredTensor(n, "<memory>", "", tuple(t.shape), 0, 0) for n, t in self.tensors.items()}
        audit(expected, stored, {n: n for n in stored}, "<memory>", ignore)

    def read(self, name: str) -> torch.Tensor:
        t = self.tensors[name]
        if t.is_floating_point():
            return t if t.dtype in (torch.float32, torch.bfloat16) else t.to(
                torch.float32 if t.dtype == torch.float64 else torch.bfloat16)
        return t.to(torch.int32)
