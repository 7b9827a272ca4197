"""Feed-forward parts: the dense gated feed-forward (SwiGLU) and the routed top-k gated experts.

  dense    out = down( act(gate n) * (up n) ), act = silu             engine/models/lfm2_moe/ref.py:180-183
  experts  logits = router(n) in 32-bit; s = sigmoid(logits); the choice is the top-k of s + expert_bias
           (the bias for the choice only); w = s[chosen], divided by (sum w + norm_floor) when normalised,
           times scale; out = sum over the chosen experts in ascending expert id of w * expert(n)
                                                                         ref.py:185-214

The gate's activation (`activation`: silu, gelu, relu2, identity) and the router's scoring function (`scoring`:
sigmoid, or softmax over all experts) are parameters of the parts' specs, passed to the kernels as codes; LFM2 uses
silu and sigmoid, and another architecture's gated or routed feed-forward reuses the same fused kernels by naming its own.

Gate and up are fused into one matrix at bind time ([2I, H], gate first), per expert for the experts
([E, 2I, H] and [E, H, I], engine/models/lfm2_moe/load.py:136-161). Experts may be stored one by one
(`<experts>.<e>.<gate|up|down>.weight`) or stacked (`<experts>.gate_up_proj [E, 2I, H]`,
`<experts>.down_proj [E, H, I]`); what the folder holds decides. Routing never leaves the device: the
plan of (row, slot) pairs sorted by expert and its tile map are built by kernels, and the expert
products skip experts nobody chose.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, register_part
from .linear import linear

@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.inter = int(spec["intermediate_size"])
        self.act = ops.activation_code(spec.get("activation", "silu"))
        self.n = {k: prefix + v for k, v in spec["names"].items()}

    def weight_specs(self, present=None):
        H, I = self.hidden_size, self.inter
        return [TensorSpec(self.n["gate"] + ".weight", (I, H)), TensorSpec(self.n["up"] + ".weight", (I, H)),
                TensorSpec(self.n["down"] + ".weight", (H, I))]

    def bind(self, read, runtime):
        self.runtime = runtime
        self.w_gate_up = torch.cat([runtime.matrix(read(self.n["gate"] + ".weight")),
                                    runtime.matrix(read(self.n["up"] + ".weight"))]).contiguous()
        self.w_down = runtime.matrix(read(self.n["down"] + ".weight"))

    def forward(self, x, step):
        act = torch.empty(x.shape[0], self.inter, dtype=x.dtype, device=x.device)
        tc = self.runtime.tensorcore
        if tc is None or not tc.gated(x, self.w_gate_up, act, self.act):      # prompts: gate, up and act(gate) * up in one kernel
            gu = linear(self.runtime, x, self.w_gate_up)
            ops.gated_mul(gu, act, self.act)
        return linear(self.runtime, act, self.w_down, out_dtype=torch.float32, defer=True)


@register_part("feed_forward", "sigmoid_topk_experts")
class SigmoidTopKExperts(Part):
    graph_safe = True

    def __init__(self, spec, prefix: str = "", hidden_size: int = 0, **_):
        super().__init__(spec, prefix, hidden_size)
        self.num_experts = int(spec["num_experts"])
        self.top_k = int(spec["top_k"])
        self.inter = int(spec["intermediate_size"])
        self.use_bias = bool(spec.get("expert_bias", True))
        self.normalize = bool(spec.get("normalize", True))
        self.scale = float(spec.get("scale", 1.0))
        self.norm_floor = float(spec.get("norm_floor", 1e-6))
        self.scoring = str(spec.get("scoring", "sigmoid"))
        ops.route_flags(self.normalize, self.scoring)          # an unknown scoring function is refused here
        self.act = ops.activation_code(spec.get("activation", "silu"))
        if not 0 < self.top_k <= self.num_experts:
            raise ValueError(f"top-{self.top_k} of {self.num_experts} experts")
        if self.num_experts > 1024 or self.top_k > 32:
            raise ValueError(f"{self.num_experts} experts top-{self.top_k}: up to 1024 experts and top-32 are implemented")
        self.n = dict(spec["names"])
        self.base = prefix + self.n["experts"]
        self._plans: dict[int, ops.MoePlan] = {}
        self._outgrown: list[ops.MoePlan] = []
        self.stacked = False
        self.load = None            # see `count_into`

    def _stacked(self, present) -> bool:
        return present is not None and (self.base + ".gate_up_proj") in present

    def weight_specs(self, present=None):
        H, I, E = self.hidden_size, self.inter, self.num_experts
        out = [TensorSpec(self.prefix + self.n["router"] + ".weight", (E, H))]
        if self.use_bias:
            out.append(TensorSpec(self.prefix + self.n["bias"], (E,), "vector", "bias"))
        self.stacked = self._stacked(present)
        if self.stacked:
            out += [TensorSpec(self.base + ".gate_up_proj", (E, 2 * I, H)), TensorSpec(self.base + ".down_proj", (E, H, I))]
        else:
            for e in range(E):
                out += [TensorSpec(f"{self.base}.{e}.{self.n['gate']}.weight", (I, H)),
                        TensorSpec(f"{self.base}.{e}.{self.n['up']}.weight", (I, H)),
                        TensorSpec(f"{self.base}.{e}.{self.n['down']}.weight", (H, I))]
        return out

    def bind(self, read, runtime):
        self.runtime = runtime
        H, I, E = self.hidden_size, self.inter, self.num_experts
        # the router's product is 32-bit in both precisions: its weights are kept in 32-bit (E x H is small)
        self.w_router = runtime.vector(read(self.prefix + self.n["router"] + ".weight"))
        self.expert_bias = runtime.vector(read(self.prefix + self.n["bias"])) if self.use_bias else None
        if self.stacked:
            self.w_gate_up = runtime.matrix(read(self.base + ".gate_up_proj"))
            self.w_down = runtime.matrix(read(self.base + ".down_proj"))
        else:
            self.w_gate_up = torch.empty(E, 2 * I, H, dtype=runtime.dtype, device=runtime.device)
            self.w_down = torch.empty(E, H, I, dtype=runtime.dtype, device=runtime.device)
            for e in range(E):
                self.w_gate_up[e, :I].copy_(read(f"{self.base}.{e}.{self.n['gate']}.weight"))
                self.w_gate_up[e, I:].copy_(read(f"{self.base}.{e}.{self.n['up']}.weight"))
                self.w_down[e].copy_(read(f"{self.base}.{e}.{self.n['down']}.weight"))

    def expected_experts_read(self, rows: int) -> float:
        """Distinct experts that `rows` rows choose when every expert is as likely as any other."""
        E, k = self.num_experts, self.top_k
        return E * (1.0 - (1.0 - k / E) ** rows)

    def step_bytes(self, elem: int, experts_read: float | None = None, rows: int = 1, **_) -> int:
        """The router (32-bit) and the expert bias, and `experts_read` experts' matrices (default: the expected number
        of distinct experts `rows` rows choose)."""
        H, I, E = self.hidden_size, self.inter, self.num_experts
        n = self.expected_experts_read(rows) if experts_read is None else experts_read
        return int(E * H * 4 + (E * 4 if self.use_bias else 0) + n * 3 * H * I * elem)

    def count_into(self, counts: torch.Tensor | None) -> None:
        """From now on every pass adds the pairs it routed to each expert to `counts` (an integer tensor [experts] on
        the device; None stops it). The adding is a kernel of the pass, so it also happens in steps replayed from CUDA
        graphs that were captured while it was on; the engine drops its graphs when it switches this."""
        self.load = counts

    def forward_from(self, norm, residual, delta, step):
        """The norm in front and this layer in one go. The router's logits are 32-bit end to end: for few rows the norm
        kernel runs the router itself on its unrounded output as it goes; for many, it also hands the unrounded rows."""
        route = self.router_args(residual.shape[0], residual.device)
        if route is not None:
            x = norm.add_norm(residual, delta, route=route)
            return self.forward(x, step, routing=(route["ids"], route["wts"]))
        x, x32 = norm.add_norm(residual, delta, want32=True)
        return self.forward(x, step, x32=x32)

    def router_args(self, rows: int, device):
        """What the norm kernel in front of the layer needs to run this layer's router on its `rows` output rows
        (for many rows the kernel norms several rows per block, so the router's weights are read once per block)."""
        return {"weight": self.w_router, "bias": self.expert_bias, "k": self.top_k, "normalize": self.normalize,
                "scoring": self.scoring, "floor": self.norm_floor, "scale": self.scale,
                "ids": torch.empty(rows, self.top_k, dtype=torch.int32, device=device),
                "wts": torch.empty(rows, self.top_k, dtype=torch.float32, device=device)}

    def route(self, x32):
        """(ids int32 [R, k], weights float32 [R, k]) of the 32-bit rows x32."""
        R = x32.shape[0]
        logits = ops.gemm_simt(x32, self.w_router, None, torch.empty(R, self.num_experts, dtype=torch.float32,
                                                                      device=x32.device))
        ids = torch.empty(R, self.top_k, dtype=torch.int32, device=x32.device)
        wts = torch.empty(R, self.top_k, dtype=torch.float32, device=x32.device)
        ops.router_topk(logits, self.expert_bias, self.top_k, self.normalize, self.norm_floor, self.scale, ids, wts,
                        self.scoring)
        return ids, wts

    def plan_for(self, pairs: int, device, tile_rows: int | None = None) -> ops.MoePlan:
        """The routing-plan buffers for up to `pairs` pairs and token tiles of `tile_rows` rows (kept and reused)."""
        tile_rows = tile_rows or ops.simt_tile_rows()
        plan = self._plans.get(tile_rows)
        if plan is None or plan.max_pairs < pairs:
            cap = max(pairs, 64) if plan is None else max(pairs, 2 * plan.max_pairs)
            if plan is not None:
                self._outgrown.append(plan)         # a captured decode graph may still use the smaller plan's buffers
            plan = self._plans[tile_rows] = ops.MoePlan(cap, self.num_experts, tile_rows, device)
        return plan

    def forward(self, x, step, x32=None, routing=None):
        """The layer's output as `ops.ExpertRows`: one 32-bit row per (row, slot) pair, which the consuming norm
        kernel weighs and adds in ascending expert id. `routing` = (ids, wts) when the norm in front already ran
        the router; else it runs here, on `x32` (the unrounded normed rows) where given."""
        R, H = x.shape[0], self.hidden_size
        ids, wts = routing if routing is not None else self.route(x32 if x32 is not None else x.float())
        if step is not None and step.trace is not None:
            step.trace.setdefault("routes", []).append((self.prefix, ids))
        tc = self.runtime.tensorcore
        if tc is not None and x.dtype == torch.bfloat16:
            rows = tc.experts(self, x, ids, wts)
            if rows is not None:
                return rows
        plan = self.plan_for(R * self.top_k, x.device).build(ids)
        if self.load is not None:
            self.load.add_(plan.counts)
        act = torch.empty(R * self.top_k, self.inter, dtype=x.dtype, device=x.device)
        ops.gemm_simt_grouped(x, plan.sorted_pairs, self.top_k, self.w_gate_up, act, plan, swiglu=self.act)
        y = torch.empty(R * self.top_k, H, dtype=torch.float32, device=x.device)
        ops.gemm_simt_grouped(act, None, 1, self.w_down, y, plan, swiglu=False)
        return ops.ExpertRows(y, plan.pos_of_pair, ids, wts)
