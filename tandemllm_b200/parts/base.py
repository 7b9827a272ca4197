"""What a part of a layer is, and the registries parts are chosen from.

A layer is put together from a mixer, a feed-forward, norms and (inside a mixer) a position encoding,
arranged by a block arrangement. Each kind is registered under a name; a `ModelSpec` names kinds and
gives every size and constant as a parameter. No part reads a model's configuration, knows the model
it is in, or knows which other parts surround it.

Interfaces (duck-typed; the base classes below document them and hold the shared plumbing):

  Norm            weight_specs() -> [TensorSpec];  bind(read, runtime);
                  add_norm(residual, delta, out=None, gather=None, n_out=None, want32=False, route=None) -> out
                                                                         residual += delta, out = norm(residual)
  PositionEncoding  fused_rotary() -> (inv_freq, rotary_dim) | None      what the fused q/k kernel can apply itself
                  apply(q, k, positions) -> None                         in place on [R, heads, D], else
  Mixer           weight_specs(present) -> [TensorSpec];  bind(read, runtime);
                  cache_need() -> PagedNeed | SlotNeed | None
                  forward(x, step, cache, writes_cache=True) -> branch output
  FeedForward     weight_specs(present);  bind(read, runtime);
                  forward(x, step) -> branch output
                  optional: forward_from(norm, residual, delta, step) -> branch output: the feed-forward runs the norm
                  in front of it itself (residual += delta, x = norm(residual)), so that what it wants from that norm
                  beyond the rounded rows (the unrounded rows, a router run inside the norm kernel) stays between the
                  two of them; `Part.forward_from` is the plain form, which an arrangement may rely on
  Arrangement     run(layer, residual, pending, step, cache, writes_cache) -> pending  (the not-yet-added branch output)

A branch output is what a mixer or feed-forward adds to the residual stream: a float32 tensor [R, hidden], or one of
the deferred forms of `kernels.ops` (`PartialSums`, `ExpertRows`) that the next norm kernel adds itself;
`kernels.ops.materialize` turns any of them into a tensor.

`step` is the `StepContext` of the running batch: rows of several requests flattened, with each row's
request, position and the request's tables and slots. `cache` is what the cache manager made for the
site from the mixer's `cache_need()`.

What a part written in torch may read of a step. The device tensors of `StepContext` are always there. `step.host`
holds host copies for launch shapes and for parts that loop in Python: `row_start` (list, B + 1) always; `start_pos`
and `slots` (lists, B) in an eager step, and None in a decode step that runs from a CUDA graph, because a replayed
graph sees new positions and slots only through the device tensors. A part that needs those host lists must leave
`graph_safe` False (the default); the step function then never captures a step that runs it.
`step.trace` is None, or a dict into which a part may put what it decided for this step (the routed feed-forward
appends (its prefix, the chosen expert ids) under "routes"); a traced step always runs eagerly.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorSpec

MIXERS: dict[str, Callable[..., Any]] = {}
FEED_FORWARDS: dict[str, Callable[..., Any]] = {}
NORMS: dict[str, Callable[..., Any]] = {}
POSITION_ENCODINGS: dict[str, Callable[..., Any]] = {}
ARRANGEMENTS: dict[str, Callable[..., Any]] = {}

_TABLES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position_encoding": POSITION_ENCODINGS,
           "arrangement": ARRANGEMENTS}


def register_part(family: str, kind: str):
    """Class decorator: make `kind` available in the `family` registry
    (mixer, feed_forward, norm, position_encoding, arrangement)."""
    table = _TABLES[family]

    def deco(cls):
        table[kind] = cls
        return cls
    return deco


def make_part(family: str, spec: PartSpec, **context):
    table = _TABLES[family]
    if spec.kind not in table:
        raise ValueError(f"unknown {family} kind {spec.kind!r}; registered: {', '.join(sorted(table)) or 'none'}")
    return table[spec.kind](spec, **context)


@dataclass
class Runtime:
    """Where and in which precision a model runs. `dtype` is the compute dtype: torch.float32 (everything in
    true 32-bit) or torch.bfloat16 (bfloat16 storage and products, 32-bit norms, softmax, router and residual)."""
    device: torch.device
    dtype: torch.dtype
    status: torch.Tensor | None = None      # int32[1] on the device: kernels record a bad index here instead of faulting
    tensorcore: Any = None                  # the bfloat16 tensor-core kernels (kernels.tensorcore.TensorCore) or None
    attention_kernels: Any = None           # faster attention kernels for bfloat16, or None: the CUDA-core kernel

    def __post_init__(self) -> None:
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype {self.dtype}: float32 and bfloat16 are implemented")
        if self.status is None and self.device.type == "cuda":
            self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def scratch(self, name: str, numel: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """A kept device buffer of at least `numel` elements for a kernel's intermediate results. Kernels on one
        stream run in order, so parts that run one after another may share a name."""
        pool = self.__dict__.setdefault("_scratch", {})
        buf = pool.get((name, dtype))
        if buf is None or buf.numel() < numel:
            if buf is not None:
                # a captured decode graph may still write to the smaller buffer: it is kept, not freed
                self.__dict__.setdefault("_outgrown", []).append(buf)
            buf = pool[(name, dtype)] = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
        return buf

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=torch.float32).contiguous()


@dataclass(frozen=True)
class PagedNeed:
    """A cache that grows with the sequence: per token, `kv_heads * head_dim` keys and as many values.
    `window`: only the last `window` positions are ever read (None: all), so pages behind it can be given back."""
    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class SlotNeed:
    """Per-request state of fixed size. When a request takes the slot it is set to `init`: None for zeros, a
    number to fill it with, or a tensor of `shape` (or broadcastable to it) that is copied in."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32
    init: Any = field(default=None, compare=False)


@dataclass
class PagedSiteCache:
    group: int                  # index of the page group (which block table to use)
    page_size: int
    k: torch.Tensor             # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor


@dataclass
class SlotSiteCache:
    state: torch.Tensor         # [slots, *shape]


@dataclass
class StepContext:
    """One batch: R rows of B requests, each request's rows consecutive and in position order."""
    n_rows: int
    n_requests: int
    token_ids: torch.Tensor         # int32 [R]
    positions: torch.Tensor         # int32 [R]  absolute position of the row's token in its sequence
    req_of_row: torch.Tensor        # int32 [R]  index into this batch's requests
    row_start: torch.Tensor         # int32 [B + 1]
    state_slot: torch.Tensor        # int32 [B]  the request's slot in every SlotSiteCache
    block_tables: list[torch.Tensor]  # per page group: int32 [B, max_pages], -1 where no page is held
    out_rows: torch.Tensor          # int32 [n_out] rows whose logits are wanted
    n_out: int
    max_rows_per_request: int = 0   # host copies, for launch shapes
    max_context: int = 0
    host: dict = field(default_factory=dict)   # host-side copies of the lists above (for parts written in torch)
    trace: dict | None = None       # when a dict: parts may record what they decided in this step (eager steps only)


class Part:
    """Shared plumbing: a part keeps its spec and names its tensors under a prefix.

    `graph_safe`: the part's forward only launches work on the current stream, with shapes that depend on the
    batch's sizes alone (no host reads of device data, no Python branches on values), so a decode step that
    runs it may be captured in a CUDA graph. A part says so itself; the default is no."""

    graph_safe = False

    def __init__(self, spec: PartSpec, prefix: str = "", hidden_size: int = 0, **_):
        self.spec = spec
        self.prefix = prefix
        self.hidden_size = hidden_size

    def weight_specs(self, present: set[str] | None = None) -> list[TensorSpec]:
        return []

    def bind(self, read: Callable[[str], torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime

    def cache_need(self):
        return None

    def step_bytes(self, elem: int, **_) -> int:
        """Bytes of this part's weights that a step reads when it uses each of them once: matrices in the compute
        dtype (`elem` bytes an element), vectors in 32-bit. Parts that read only some of their weights in a step
        (routed experts) answer for themselves; nested parts (a mixer's norms) are counted by their owner."""
        total = 0
        for spec in self.weight_specs(None):
            n = 1
            for d in spec.shape:
                n *= d
            total += n * (elem if spec.role == "matrix" else 4)
        return total

    def forward_from(self, norm, residual: torch.Tensor, delta, step: "StepContext"):
        """A feed-forward behind its norm: residual += delta, x = norm(residual), the branch output of x."""
        return self.forward(norm.add_norm(residual, delta), step)
