"""RMS norm fused with the residual add in front of it.

  y = x * rsqrt(mean(x^2) + eps);  out = w * y      plain w, not 1 + w  (engine/models/lfm2_moe/ref.py:105-109)

The residual stream is 32-bit; mean, rsqrt and the scale are 32-bit and the result is rounded once to the
compute dtype. The reference fuses the same pair (`add_rms`, engine/models/lfm2_moe/kernels.py:90-107).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", size: int = 0, **_):
        super().__init__(spec, prefix)
        self.size = size
        self.eps = float(spec["eps"])
        self.name = prefix + "weight"
        self.weight = None

    def weight_specs(self, present=None):
        return [TensorSpec(self.name, (self.size,), role="vector", init="ones")]

    def bind(self, read, runtime):
        self.runtime = runtime
        self.weight = runtime.vector(read(self.name))

    def add_norm(self, residual: torch.Tensor, delta, out: torch.Tensor | None = None,
                 gather: torch.Tensor | None = None, n_out: int | None = None, want32: bool = False,
                 route: dict | None = None):
        """residual += delta (32-bit; a tensor or a branch output in one of the deferred forms of `kernels.ops`);
        returns the normed rows in the compute dtype, and with `want32` the pair (normed, the same rows unrounded
        in 32-bit). `route` (see `ops.add_rmsnorm`) also runs a router on the unrounded rows in the same kernel."""
        rows = residual.shape[0] if gather is None else (n_out if n_out is not None else gather.shape[0])
        if out is None:
            out = torch.empty(rows, self.size, dtype=self.runtime.dtype, device=residual.device)
        if not want32:
            return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, gather, None, route)
        if out.dtype == torch.float32:
            ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, gather, None, route)
            return out, out
        out32 = torch.empty(rows, self.size, dtype=torch.float32, device=residual.device)
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, gather, out32, route)
        return out, out32
