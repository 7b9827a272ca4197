"""The double-gated short-convolution mixer with a fixed-size per-request state.

  bcx = in_proj(n); B, C, x = thirds of bcx; bx = B * x; conv over the last `taps` inputs bx of the
  sequence (causal, depthwise, tap taps-1 multiplies the row itself); y = C * conv; out = out_proj(y);
  the state after a step is the last taps-1 inputs bx; a new sequence starts from zeros
  (engine/models/lfm2_moe/ref.py:134-151, :253).

With `bias` the three bias vectors are bound as `<in>.bias [3H]`, `<taps>.bias [H]` (added to the tap sum
before the C gate) and `<out>.bias [H]`; the reference implements the bias-free form only
(engine/models/lfm2_moe/config.py:47).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, SlotNeed, register_part
from .linear import linear


@register_part("mixer", "short_conv")
class ShortConvMixer(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.taps = int(spec["taps"])
        if not 2 <= self.taps <= 16:
            raise ValueError(f"short conv with {self.taps} taps: 2 to 16 are implemented")
        self.bias = bool(spec.get("bias", False))
        self.n = {k: prefix + v for k, v in spec["names"].items()}

    def weight_specs(self, present=None):
        H, K = self.hidden_size, self.taps
        out = [TensorSpec(self.n["in"] + ".weight", (3 * H, H)), TensorSpec(self.n["taps"] + ".weight", (H, 1, K), "vector"),
               TensorSpec(self.n["out"] + ".weight", (H, H))]
        if self.bias:
            out += [TensorSpec(self.n["in"] + ".bias", (3 * H,), "vector", "bias"),
                    TensorSpec(self.n["taps"] + ".bias", (H,), "vector", "bias"),
                    TensorSpec(self.n["out"] + ".bias", (H,), "vector", "bias")]
        return out

    def bind(self, read, runtime):
        self.runtime = runtime
        H, K = self.hidden_size, self.taps
        self.w_in = runtime.matrix(read(self.n["in"] + ".weight"))
        self.w_out = runtime.matrix(read(self.n["out"] + ".weight"))
        self.w_taps = runtime.vector(read(self.n["taps"] + ".weight")).reshape(H, K).contiguous()
        self.b_in = self.b_taps = self.b_out = None
        if self.bias:
            self.b_in = runtime.vector(read(self.n["in"] + ".bias"))
            self.b_taps = runtime.vector(read(self.n["taps"] + ".bias"))
            self.b_out = runtime.vector(read(self.n["out"] + ".bias"))

    def cache_need(self):
        return SlotNeed((self.taps - 1, self.hidden_size), torch.float32)

    def forward(self, x, step, cache, writes_cache: bool = True):
        H = self.hidden_size
        y = torch.empty(x.shape[0], H, dtype=x.dtype, device=x.device)
        if step.max_rows_per_request == 1:
            # decoding. A handful of rows: the in-projection's kernel convolves and shifts the state in its epilogue.
            # More: one kernel convolves and shifts the state, and adds the projection's partial sums itself.
            tc = self.runtime.tensorcore
            if tc is None or not tc.in_proj_conv(x, self.w_in, self.b_in, self.w_taps, self.b_taps, cache.state,
                                                 step.state_slot, step.req_of_row, step.positions, y, writes_cache):
                bcx = linear(self.runtime, x, self.w_in, self.b_in, defer="rounded")
                ops.short_conv_decode(bcx, self.w_taps, self.b_taps, cache.state, step.state_slot, step.req_of_row,
                                      step.positions, y, write_state=writes_cache)
            return linear(self.runtime, y, self.w_out, self.b_out, out_dtype=torch.float32, defer=True)
        bcx = linear(self.runtime, x, self.w_in, self.b_in)
        ops.short_conv(bcx, self.w_taps, self.b_taps, cache.state, step.state_slot, step.req_of_row, step.row_start,
                       step.positions, y)
        if writes_cache:
            ops.short_conv_state(bcx, cache.state, step.state_slot, step.row_start, step.positions, step.n_requests,
                                 H, self.taps)
        return linear(self.runtime, y, self.w_out, self.b_out, out_dtype=torch.float32, defer=True)
