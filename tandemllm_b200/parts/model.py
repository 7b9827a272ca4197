"""The decoder built from a `ModelSpec`: embedding, the scheduled layers, final norm, head.

  h = embed[tokens]; for each site of the schedule: run its layer on its cache; h = final_norm(h);
  logits = h @ head^T in 32-bit, head = the embedding when tied   (engine/models/lfm2_moe/ref.py:218-241)

The model owns no cache: `cache_needs()` tells the cache manager what every site needs and `forward` is
given the per-site caches it made. It computes the final norm and the head for the wanted rows only.
"""

from __future__ import annotations

import torch

from ..config.spec import ModelSpec
from ..kernels import ops
from ..settings import SETTINGS
from ..weights.loader import TensorSpec
from .base import Runtime, StepContext, make_part
from .block import Layer
from .linear import linear


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.hidden_size, self.vocab_size = spec.hidden_size, spec.vocab_size
        self.layers = [Layer(ls, spec.hidden_size) for ls in spec.layers]
        self.final_norm = make_part("norm", spec.final_norm, prefix=spec.final_norm_prefix, size=spec.hidden_size)
        self.runtime: Runtime | None = None
        self.embedding = self.head = None

    # ---- weights ----
    def weight_specs(self, present: set[str] | None = None) -> list[TensorSpec]:
        s = self.spec
        out = [TensorSpec(s.embedding_name, (s.vocab_size, s.hidden_size))]
        out += self.final_norm.weight_specs(present)
        if s.head_name:
            out.append(TensorSpec(s.head_name, (s.vocab_size, s.hidden_size)))
        for layer in self.layers:
            out += layer.weight_specs(present)
        return out

    def load(self, weights, runtime: Runtime) -> "DecoderModel":
        """Check `weights` (a FolderWeights or DictWeights) against what the parts read, then bind every part."""
        s = self.spec
        present = weights.present()
        specs = self.weight_specs(present)
        ignored = set(s.ignored_names)
        weights.check(specs, ignore=(lambda n: n in ignored) if ignored else None)
        self.runtime = runtime
        self.embedding = runtime.matrix(weights.read(s.embedding_name))
        self.head = runtime.matrix(weights.read(s.head_name)) if s.head_name else self.embedding
        self.final_norm.bind(weights.read, runtime)
        for layer in self.layers:
            layer.bind(weights.read, runtime)
        return self

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for obj in [self, self.final_norm] + [p for layer in self.layers for p in layer.parts]:
            stack = [obj]
            while stack:
                o = stack.pop()
                for v in vars(o).values():
                    if isinstance(v, torch.Tensor) and v.is_cuda and v.data_ptr() not in seen:
                        seen.add(v.data_ptr())
                        total += v.numel() * v.element_size()
                    elif hasattr(v, "weight_specs") and v is not o:
                        stack.append(v)
        return total

    def decode_bytes(self, batch: int, experts_read: list[float] | None = None) -> dict:
        """Bytes of weights one decode step of `batch` rows reads, every weight it uses once (the reference accounts a
        token the same way, engine/models/lfm2_moe/pack.py:292-315): per site of the run order its norms', mixer's and
        feed-forward's weights as the parts themselves count them (`Part.step_bytes`), the last norm, the head, and
        `batch` rows of the embedding. `experts_read[i]`: the experts the i-th routed site of the run order really
        read (default: what uniform routing of `batch` rows would). The cache's bytes are the engine's to add."""
        elem = torch.empty(0, dtype=self.runtime.dtype).element_size() if self.runtime else 2
        it = iter(experts_read) if experts_read is not None else None
        dense = experts = 0
        for site in self.spec.schedule:
            layer = self.layers[site.layer]
            for part in layer.parts:
                if hasattr(part, "expected_experts_read"):
                    n = next(it) if it is not None else None
                    whole = part.step_bytes(elem, experts_read=n, rows=batch)
                    fixed = part.step_bytes(elem, experts_read=0)
                    dense += fixed
                    experts += whole - fixed
                else:
                    dense += part.step_bytes(elem)
        dense += self.final_norm.step_bytes(elem)
        head = self.vocab_size * self.hidden_size * elem
        embed = batch * self.hidden_size * elem
        return {"dense": dense, "experts": experts, "head": head, "embedding_rows": embed,
                "total": dense + experts + head + embed}

    @property
    def graph_safe(self) -> bool:
        """Every part of every layer says its forward may be captured in a CUDA graph."""
        return all(getattr(p, "graph_safe", False) for layer in self.layers for p in layer.parts) and \
            getattr(self.final_norm, "graph_safe", False)

    # ---- caches ----
    def cache_needs(self) -> list:
        """Per site of the schedule: the need of its mixer, or None when the site reads another site's cache."""
        return [None if site.cache_of is not None else self.layers[site.layer].mixer.cache_need()
                for site in self.spec.schedule]

    # ---- the forward pass of one batch ----
    def forward(self, step: StepContext, site_caches: list) -> torch.Tensor:
        rt = self.runtime
        residual = torch.empty(step.n_rows, self.hidden_size, dtype=torch.float32, device=rt.device)
        ops.embed_rows(self.embedding, step.token_ids, residual, rt.status)
        pending = None
        ranges = SETTINGS.is_set("NVTX")             # named ranges for profilers: the step, and each layer in run order
        if ranges:
            torch.cuda.nvtx.range_push(f"step rows={step.n_rows} requests={step.n_requests}")
        try:
            for i, site in enumerate(self.spec.schedule):
                own = site.cache_of is None
                cache = site_caches[i if own else site.cache_of]
                if ranges:
                    layer = self.layers[site.layer]
                    torch.cuda.nvtx.range_push(f"site {i} layer {site.layer} {type(layer.mixer).__name__} + "
                                               f"{type(layer.feed_forward).__name__}")
                pending = self.layers[site.layer].run(residual, pending, step, cache, writes_cache=own)
                if ranges:
                    torch.cuda.nvtx.range_pop()
            if step.n_out == 0:
                return torch.empty(0, self.vocab_size, dtype=torch.float32, device=rt.device)
            if ranges:
                torch.cuda.nvtx.range_push("final norm + head")
            n = self.final_norm.add_norm(residual, pending, gather=step.out_rows, n_out=step.n_out)
            out = linear(rt, n, self.head, out_dtype=torch.float32)
            if ranges:
                torch.cuda.nvtx.range_pop()
            return out
        finally:
            if ranges:
                torch.cuda.nvtx.range_pop()
