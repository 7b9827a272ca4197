"""Sampling options of a request, and the batched draw on the device.

Options and their meaning are the reference's (`Sampler`, engine/sample.py:103-131): `temperature` 0 is
greedy whatever the filters say (sample.py:134-141); otherwise logits / temperature, then `min_p`, then
`top_k`, then `top_p` (sample.py:172-199), then a draw. A draw is Gumbel-max with noise keyed by
(seed, sequence position) (sample.py:311-322), so a seeded request yields the same tokens whatever shares
its batch; a request without a seed takes one from the operating system when it is made (sample.py:164-169).

One kernel launch draws for every row of a step (`kernels.ops.sample`); a step of greedy rows only uses
the argmax kernel.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from ..kernels import ops


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: int | None = None
    max_tokens: int = 128           # new tokens at most
    stop_token_ids: tuple[int, ...] | None = None    # None: the model's own stop ids
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if self.temperature < 0.0 or self.temperature != self.temperature:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be at least 1, got {self.max_tokens}")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    def resolved_seed(self) -> int:
        """The request's seed as a 63-bit integer; an unseeded request draws one now."""
        if self.seed is None:
            self.seed = int.from_bytes(os.urandom(8), "little") >> 1
        return int(self.seed) & ((1 << 63) - 1)


class Sampler:
    """Draws one token per logits row on the device. Rows are (params, position) pairs: `position` is the
    index in the sequence of the token being drawn."""

    def __init__(self, device):
        self.device = device
        self._cap = 0

    def _staging(self, n: int):
        """A pinned block and its device copy for n rows. Three pairs take turns, each waiting only for the copy that last
        read it, so that a step can be launched while the one before it still runs."""
        if n > self._cap:
            self._cap = max(64, 2 * n)
            # one pinned block: temperature, top_p, min_p (float32) | top_k, position (int32) | seed (int64)
            self._hosts = [torch.empty(7 * self._cap, dtype=torch.int32, pin_memory=True) for _ in range(3)]
            self._devs = [torch.empty(7 * self._cap, dtype=torch.int32, device=self.device) for _ in range(3)]
            self._events = [None, None, None]
            self._turn = 0
        self._turn = (self._turn + 1) % 3
        if self._events[self._turn] is not None:
            self._events[self._turn].synchronize()
        return self._hosts[self._turn], self._devs[self._turn]

    def __call__(self, logits: torch.Tensor, rows: list[tuple[SamplingParams, int]]) -> torch.Tensor:
        """int32 [n] token ids for float32 logits [n, V]."""
        n = logits.shape[0]
        if n != len(rows):
            raise ValueError(f"{n} logits rows for {len(rows)} requests")
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
        if n == 0:
            return out
        if all(p.greedy for p, _ in rows):
            return ops.argmax(logits, out)
        host, dev = self._staging(n)
        c = self._cap
        f = host.view(torch.float32)
        seeds = host[5 * c:7 * c].view(torch.int64)
        for i, (p, pos) in enumerate(rows):
            f[i] = p.temperature
            f[c + i] = p.top_p
            f[2 * c + i] = p.min_p
            host[3 * c + i] = p.top_k
            host[4 * c + i] = pos
            seeds[i] = p.resolved_seed() if not p.greedy else 0
        dev.copy_(host, non_blocking=True)
        event = self._events[self._turn] or torch.cuda.Event()
        event.record()
        self._events[self._turn] = event
        df = dev.view(torch.float32)
        return ops.sample(logits, df[0:n], dev[3 * c:3 * c + n], df[c:c + n], df[2 * c:2 * c + n],
                          dev[5 * c:7 * c].view(torch.int64)[:n], dev[4 * c:4 * c + n], out)
