"""Position encodings applied to q and k inside a mixer.

`rope_neox`: inv_freq_i = theta^(-2i/d), angle = position * inv_freq_i (32-bit), the two halves of the
rotated part share a frequency: x' = x cos + rotate_half(x) sin with rotate_half(x) = cat(-x[d/2:], x[:d/2])
(engine/models/lfm2_moe/ref.py:84, 111-120). The frequencies are computed here once, in 32-bit, by the
reference's expression; the angles, sines and cosines are computed in the kernel in 32-bit per row.

`none`: q and k are left as they are.

An encoding either hands the fused q/k kernel its table (`fused_rotary`), or is applied by the mixer
through `apply(q, k, positions)` between the norm and the cache write.
"""

from __future__ import annotations

import torch

from .base import Part, register_part


@register_part("position_encoding", "rope_neox")
class RotaryNeox(Part):
    graph_safe = True

    def __init__(self, spec, head_dim: int = 0, **_):
        super().__init__(spec)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec.get("rotary_dim") or head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} for head size {head_dim}: an even size up to the head size")
        self.inv_freq = None

    def bind(self, read, runtime):
        self.runtime = runtime
        d = self.rotary_dim
        inv = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        self.inv_freq = inv.to(runtime.device)

    def fused_rotary(self):
        return self.inv_freq, self.rotary_dim

    def apply(self, q, k, positions):
        raise NotImplementedError("rope_neox is applied by the fused q/k kernel")


@register_part("position_encoding", "none")
class NoPosition(Part):
    graph_safe = True

    def __init__(self, spec, head_dim: int = 0, **_):
        super().__init__(spec)

    def fused_rotary(self):
        return None, 0

    def apply(self, q, k, positions):
        return None
