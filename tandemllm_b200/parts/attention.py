"""The attention mixer: grouped-query attention over the paged cache with optional per-head q/k RMS norms,
a position encoding, and an optional sliding window.

  q = norm_D(q_proj n), k = norm_D(k_proj n), v = v_proj n; position encoding on q, k; k, v written to the
  cache at the row's position; s = q k^T * scale over the visible keys; softmax in 32-bit; o = a v;
  query head h reads KV head h // (Hq / Hk); out = out_proj(o)      (engine/models/lfm2_moe/ref.py:153-178)

Every size (heads, KV heads, head size), the scale, the window and the names of its tensors are
parameters. The q, k and v matrices are fused into one product at bind time, as the reference's loader
does (engine/models/lfm2_moe/load.py:125-135). A site that reads another site's cache computes its own
q and attends over the keys and values the other site wrote.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import PagedNeed, Part, make_part, register_part
from .linear import linear

@register_part("mixer", "attention")
class AttentionMixer(Part):
    @property
    def graph_safe(self) -> bool:
        return self.position.graph_safe

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} query heads are not a multiple of {self.num_kv_heads} KV heads")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"head size {self.head_dim}: multiples of 16 from 16 to 256 are implemented")
        self.scale = float(spec.get("scale") or self.head_dim ** -0.5)
        self.window = spec.get("window")
        names = spec["names"]
        self.n = {k: prefix + v for k, v in names.items()}
        qk = spec.get("qk_norm")
        self.q_norm = make_part("norm", qk, prefix=self.n["q_norm"] + ".", size=self.head_dim) if qk else None
        self.k_norm = make_part("norm", qk, prefix=self.n["k_norm"] + ".", size=self.head_dim) if qk else None
        self.position = make_part("position_encoding", spec["position"], head_dim=self.head_dim)
        self.bias = bool(spec.get("bias", False))

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    def weight_specs(self, present=None):
        H = self.hidden_size
        out = [TensorSpec(self.n["q"] + ".weight", (self.q_dim, H)), TensorSpec(self.n["k"] + ".weight", (self.kv_dim, H)),
               TensorSpec(self.n["v"] + ".weight", (self.kv_dim, H)), TensorSpec(self.n["out"] + ".weight", (H, self.q_dim))]
        if self.q_norm:
            out += self.q_norm.weight_specs() + self.k_norm.weight_specs()
        return out

    def bind(self, read, runtime):
        self.runtime = runtime
        self.w_qkv = torch.cat([runtime.matrix(read(self.n[x] + ".weight")) for x in ("q", "k", "v")]).contiguous()
        self.w_out = runtime.matrix(read(self.n["out"] + ".weight"))
        if self.q_norm:
            self.q_norm.bind(read, runtime)
            self.k_norm.bind(read, runtime)
        self.position.bind(read, runtime)

    def cache_need(self):
        return PagedNeed(self.num_kv_heads, self.head_dim, self.window)

    def forward(self, x, step, cache, writes_cache: bool = True):
        R, dt, dev = x.shape[0], x.dtype, x.device
        Hq, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        status = self.runtime.status
        qkv = linear(self.runtime, x, self.w_qkv)
        q = torch.empty(R, Hq, D, dtype=dt, device=dev)
        table = step.block_tables[cache.group]
        qw = self.q_norm.weight if self.q_norm else None
        kw = self.k_norm.weight if self.k_norm else None
        eps = self.q_norm.eps if self.q_norm else 0.0
        fused = self.position.fused_rotary()
        if fused is not None and writes_cache:
            inv_freq, rot = fused
            ops.qk_prepare(qkv, qw, kw, eps, inv_freq, rot, step.positions, step.req_of_row, table, cache.page_size,
                           q, cache.k, cache.v, None, None, Hq, Hk, D, status)
        else:
            k = torch.empty(R, Hk, D, dtype=dt, device=dev)
            v = torch.empty(R, Hk, D, dtype=dt, device=dev)
            inv_freq, rot = fused if fused is not None else (None, 0)
            ops.qk_prepare(qkv, qw, kw, eps, inv_freq, rot, step.positions, step.req_of_row, None, 0,
                           q, None, None, k, v, Hq, Hk, D, status)
            if fused is None:
                self.position.apply(q, k, step.positions)
            if writes_cache:
                ops.kv_store(k, v, step.positions, step.req_of_row, table, cache.page_size, cache.k, cache.v, status)
        o = torch.empty(R, Hq, D, dtype=dt, device=dev)
        fast = self.runtime.attention_kernels
        if fast is None or not fast.attention(q, cache, table, step, self.scale, self.window, o, self.runtime):
            spans = ops.attention_spans(step.max_context)
            scratch = self.runtime.scratch("attention", ops.attention_scratch_floats(R, Hq, D, spans))
            ops.paged_attention_split(q, cache.k, cache.v, table, cache.page_size, step.req_of_row, step.positions,
                                      self.scale, self.window, o, scratch, spans, status)
        return linear(self.runtime, o.view(R, Hq * D), self.w_out, out_dtype=torch.float32, defer=True)
