"""Each part alone against the plain implementation's function for it, and the generality of the parts: a toy
mixer with state of its own, defined here, is registered, built into a model with a windowed attention layer, a
layer that runs twice and a site that reads another site's cache, and stepped, without a change to the package.
"""

import json
import types

import pytest
import torch

from tests import plain_lfm2 as P
from tests.helpers import max_rel

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runtime(dtype=torch.float32):
    from tandemllm_b200.parts import Runtime
    return Runtime(torch.device(DEV), dtype)


def stepper(needs, rt, pages=64, requests=4, page=16):
    """A cache manager for the given site needs and a function that turns (request, tokens) lists into the
    StepContext of a batch, advancing the requests as the step function does."""
    from tandemllm_b200.cache import CacheManager
    from tandemllm_b200.engine.step import StepEntry, StepFunction
    cache = CacheManager(needs, num_pages=pages, max_requests=requests, page_size=page, dtype=rt.dtype, device=rt.device)
    fn = StepFunction(types.SimpleNamespace(runtime=rt, vocab_size=1), cache, check_status=False)

    def step(batch):
        for rid, _ in batch:
            if not cache.has(rid):
                cache.admit(rid)
        ctx = fn.build([StepEntry(rid, list(range(n)), []) for rid, n in batch])
        for rid, n in batch:
            cache.advance(rid, cache.length_of(rid) + n)
        return ctx
    return cache, step


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def plain(branch) -> torch.Tensor:
    """A part's output on the CPU as a plain tensor, whatever form the part returned it in."""
    from tandemllm_b200.kernels import ops
    return ops.materialize(branch).cpu()


def reader(W):
    return lambda name: W[name]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_attention_part_alone(dtype, tol):
    from tandemllm_b200.config import PartSpec
    from tandemllm_b200.parts import make_part
    H, Hq, Hk, D, T = 80, 6, 3, 32, 45
    cfg = dict(num_attention_heads=Hq, num_key_value_heads=Hk, head_dim=D, hidden_size=H, norm_eps=1e-5, rope_theta=3e4)
    W = {"a.q_proj.weight": rnd(Hq * D, H, seed=1, scale=0.2), "a.k_proj.weight": rnd(Hk * D, H, seed=2, scale=0.2),
         "a.v_proj.weight": rnd(Hk * D, H, seed=3, scale=0.2), "a.out_proj.weight": rnd(H, Hq * D, seed=4, scale=0.2),
         "a.q_layernorm.weight": 1 + rnd(D, seed=5, scale=0.1), "a.k_layernorm.weight": 1 + rnd(D, seed=6, scale=0.1)}
    W = {k: v.to(dtype).float() for k, v in W.items()}
    spec = PartSpec("attention", {"num_heads": Hq, "num_kv_heads": Hk, "head_dim": D,
                                  "qk_norm": PartSpec("rmsnorm", {"eps": 1e-5}),
                                  "position": PartSpec("rope_neox", {"theta": 3e4, "rotary_dim": D}), "window": None,
                                  "names": {"q": "q_proj", "k": "k_proj", "v": "v_proj", "out": "out_proj",
                                            "q_norm": "q_layernorm", "k_norm": "k_layernorm"}})
    rt = runtime(dtype)
    part = make_part("mixer", spec, prefix="a.", hidden_size=H)
    assert {s.name for s in part.weight_specs()} == set(W)
    part.bind(reader(W), rt)
    cache, step = stepper([part.cache_need()], rt)
    x = rnd(T, H, seed=7).to(dtype)
    want = P.attention(x.float(), W, "a.", cfg)
    outs = []
    for lo, hi in ((0, 17), (17, 18), (18, T)):
        ctx = step([("r", hi - lo)])
        outs.append(plain(part.forward(x[lo:hi].to(DEV), ctx, cache.site_cache[0])))
    assert max_rel(torch.cat(outs), want) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("bias", [False, True])
def test_short_conv_part_alone(dtype, tol, bias):
    from tandemllm_b200.config import PartSpec
    from tandemllm_b200.parts import make_part
    H, K, T = 72, 4, 30
    W = {"c.in_proj.weight": rnd(3 * H, H, seed=1, scale=0.3), "c.conv.weight": rnd(H, 1, K, seed=2, scale=0.5),
         "c.out_proj.weight": rnd(H, H, seed=3, scale=0.3)}
    if bias:
        W.update({"c.in_proj.bias": rnd(3 * H, seed=4, scale=0.2), "c.conv.bias": rnd(H, seed=5, scale=0.2),
                  "c.out_proj.bias": rnd(H, seed=6, scale=0.2)})
    W = {k: v.to(dtype).float() for k, v in W.items()}
    spec = PartSpec("short_conv", {"taps": K, "bias": bias, "names": {"in": "in_proj", "taps": "conv", "out": "out_proj"}})
    rt = runtime(dtype)
    part = make_part("mixer", spec, prefix="c.", hidden_size=H)
    assert {s.name for s in part.weight_specs()} == set(W)
    part.bind(reader(W), rt)
    cache, step = stepper([part.cache_need()], rt)
    x = rnd(T, H, seed=7).to(dtype)
    want = P.short_conv(x.float(), W, "c.", K, bias)
    outs = []
    for lo, hi in ((0, 2), (2, 3), (3, 4), (4, 21), (21, T)):
        ctx = step([("r", hi - lo)])
        outs.append(plain(part.forward(x[lo:hi].to(DEV), ctx, cache.site_cache[0])))
    assert max_rel(torch.cat(outs), want) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_feed_forward_parts_alone(dtype, tol):
    from tandemllm_b200.config import PartSpec
    from tandemllm_b200.parts import make_part
    H, I, E, k, Im, T = 72, 100, 6, 3, 40, 50
    rt = runtime(dtype)
    W = {"f.w1.weight": rnd(I, H, seed=1, scale=0.2), "f.w3.weight": rnd(I, H, seed=2, scale=0.2),
         "f.w2.weight": rnd(H, I, seed=3, scale=0.2)}
    W = {k_: v.to(dtype).float() for k_, v in W.items()}
    dense = make_part("feed_forward", PartSpec("swiglu", {"intermediate_size": I, "names": {"gate": "w1", "up": "w3", "down": "w2"}}),
                      prefix="f.", hidden_size=H)
    dense.bind(reader(W), rt)
    x = rnd(T, H, seed=4).to(dtype)
    assert max_rel(plain(dense.forward(x.to(DEV), None)), P.dense_mlp(x.float(), W, "f.")) < tol
    for use_bias, normalize, scale in ((True, True, 1.0), (False, False, 2.0)):
        M = {"m.gate.weight": rnd(E, H, seed=5, scale=0.5), "m.expert_bias": rnd(E, seed=6, scale=0.3)}
        for e in range(E):
            M[f"m.experts.{e}.w1.weight"] = rnd(Im, H, seed=10 + e, scale=0.2)
            M[f"m.experts.{e}.w3.weight"] = rnd(Im, H, seed=30 + e, scale=0.2)
            M[f"m.experts.{e}.w2.weight"] = rnd(H, Im, seed=50 + e, scale=0.2)
        if not use_bias:
            del M["m.expert_bias"]
        M = {k_: (v if k_.endswith("expert_bias") else v.to(dtype).float()) for k_, v in M.items()}
        spec = PartSpec("sigmoid_topk_experts", {"num_experts": E, "top_k": k, "intermediate_size": Im,
                                                 "expert_bias": use_bias, "normalize": normalize, "scale": scale,
                                                 "names": {"router": "gate", "bias": "expert_bias", "experts": "experts",
                                                           "gate": "w1", "up": "w3", "down": "w2"}})
        part = make_part("feed_forward", spec, prefix="m.", hidden_size=H)
        assert {s.name for s in part.weight_specs(set(M))} == set(M)
        part.bind(reader(M), rt)
        cfg = dict(num_experts_per_tok=k, use_expert_bias=use_bias, norm_topk_prob=normalize, routed_scaling_factor=scale)
        margins = P.routing_margin(x.float(), M, "m.", cfg)
        got = plain(part.forward(x.to(DEV), None, x32=x.float().to(DEV)))
        want = P.moe(x.float(), M, "m.", cfg)
        stable = margins > 1e-4
        assert int(stable.sum()) > T // 2
        assert max_rel(got[stable], want[stable]) < tol


def test_norm_part_alone():
    from tandemllm_b200.config import PartSpec
    from tandemllm_b200.parts import make_part
    H = 100
    W = {"n.weight": 1 + rnd(H, seed=1, scale=0.3)}
    part = make_part("norm", PartSpec("rmsnorm", {"eps": 1e-3}), prefix="n.", size=H)
    part.bind(reader(W), runtime(torch.bfloat16))
    res, delta = rnd(9, H, seed=2), rnd(9, H, seed=3)
    r = res.clone().to(DEV)
    out, out32 = part.add_norm(r, delta.to(DEV), want32=True)
    want = P.rms_norm(res + delta, W["n.weight"], 1e-3)
    assert max_rel(out32.cpu(), want) < 1e-5 and max_rel(out.float().cpu(), want) < 1e-2
    assert max_rel(r.cpu(), res + delta) < 1e-6


# ------------------------------------------------------------------------------------------ a toy architecture
def register_toy():
    """A mixer with state of its own (a per-channel running sum with decay), registered from the test."""
    from tandemllm_b200.parts import Part, SlotNeed, register_part
    from tandemllm_b200.weights.loader import TensorSpec

    @register_part("mixer", "toy_decay")
    class ToyDecay(Part):
        def __init__(self, spec, prefix="", hidden_size=0, **_):
            super().__init__(spec, prefix, hidden_size)
            self.name = prefix + spec["name"]

        def weight_specs(self, present=None):
            return [TensorSpec(self.name, (self.hidden_size,), role="vector", init="bias")]

        def bind(self, read, runtime):
            self.runtime = runtime
            self.decay = torch.sigmoid(runtime.vector(read(self.name)))

        def cache_need(self):
            return SlotNeed((self.hidden_size,), torch.float32)

        def forward(self, x, step, cache, writes_cache=True):
            out = torch.empty(x.shape[0], self.hidden_size, dtype=torch.float32, device=x.device)
            starts, slots, first = step.host["row_start"], step.host["slots"], step.host["start_pos"]
            for b in range(step.n_requests):
                s = cache.state[slots[b]].clone() if first[b] > 0 else torch.zeros_like(cache.state[slots[b]])
                for r in range(starts[b], starts[b + 1]):
                    s = self.decay * s + x[r].float()
                    out[r] = s
                if writes_cache:
                    cache.state[slots[b]] = s
            return out
    return ToyDecay


def register_toy_switch_and_position():
    """A feed-forward with routing of its own (the one expert with the largest router logit, unweighted) and another
    position encoding (rotation of interleaved pairs, applied by the mixer between the norm and the cache write)."""
    from tandemllm_b200.parts import Part, register_part
    from tandemllm_b200.parts.linear import linear
    from tandemllm_b200.weights.loader import TensorSpec

    @register_part("feed_forward", "toy_switch")
    class ToySwitch(Part):
        def __init__(self, spec, prefix="", hidden_size=0, **_):
            super().__init__(spec, prefix, hidden_size)
            self.experts, self.inner = int(spec["experts"]), int(spec["inner"])

        def weight_specs(self, present=None):
            H, I = self.hidden_size, self.inner
            out = [TensorSpec(self.prefix + "switch.weight", (self.experts, H))]
            for e in range(self.experts):
                out += [TensorSpec(f"{self.prefix}e{e}.up.weight", (I, H)), TensorSpec(f"{self.prefix}e{e}.down.weight", (H, I))]
            return out

        def bind(self, read, runtime):
            self.runtime = runtime
            self.w_switch = runtime.matrix(read(self.prefix + "switch.weight"))
            self.w = [(runtime.matrix(read(f"{self.prefix}e{e}.up.weight")), runtime.matrix(read(f"{self.prefix}e{e}.down.weight")))
                      for e in range(self.experts)]

        def forward(self, x, step, x32=None, routing=None):
            choice = linear(self.runtime, x, self.w_switch, out_dtype=torch.float32).argmax(-1)
            out = torch.zeros(x.shape[0], self.hidden_size, dtype=torch.float32, device=x.device)
            for e, (up, down) in enumerate(self.w):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    hidden = torch.relu(linear(self.runtime, x[rows].contiguous(), up))
                    out[rows] = linear(self.runtime, hidden, down, out_dtype=torch.float32)
            return out

    @register_part("position_encoding", "toy_pairs")
    class ToyPairs(Part):
        def __init__(self, spec, head_dim=0, **_):
            super().__init__(spec)
            self.step_angle = float(spec["angle"])

        def bind(self, read, runtime):
            self.runtime = runtime

        def fused_rotary(self):
            return None                                             # not something the fused q/k kernel applies

        def apply(self, q, k, positions):
            ang = positions.float()[:, None, None] * self.step_angle
            cos, sin = torch.cos(ang), torch.sin(ang)
            for t in (q, k):                                        # in place: pair (2i, 2i+1) turns by position * angle
                a, b = t[..., 0::2].float().clone(), t[..., 1::2].float().clone()
                t[..., 0::2] = (a * cos - b * sin).to(t.dtype)
                t[..., 1::2] = (a * sin + b * cos).to(t.dtype)
    return ToySwitch, ToyPairs


def toy_spec(raw):
    from tandemllm_b200.config import ModelSpec, PartSpec, Site
    from tandemllm_b200.config.spec import LayerSpec
    H, eps = raw["width"], raw["eps"]
    norm = lambda name: PartSpec("rmsnorm", {"eps": eps, "name": name})
    ffn = PartSpec("swiglu", {"intermediate_size": raw["inner"], "names": {"gate": "w1", "up": "w3", "down": "w2"}})
    attn = PartSpec("attention", {"num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                  "qk_norm": PartSpec("rmsnorm", {"eps": eps}),
                                  "position": PartSpec("rope_neox", {"theta": 1e4, "rotary_dim": 16}),
                                  "window": raw["window"],
                                  "names": {"q": "q_proj", "k": "k_proj", "v": "v_proj", "out": "out_proj",
                                            "q_norm": "q_layernorm", "k_norm": "k_layernorm"}})
    toy = PartSpec("toy_decay", {"name": "decay"})
    turned = PartSpec("attention", {"num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                    "qk_norm": PartSpec("rmsnorm", {"eps": eps}),
                                    "position": PartSpec("toy_pairs", {"angle": 0.37}), "window": None,
                                    "names": {"q": "q_proj", "k": "k_proj", "v": "v_proj", "out": "out_proj",
                                              "q_norm": "q_layernorm", "k_norm": "k_layernorm"}})
    switch = PartSpec("toy_switch", {"experts": 3, "inner": 40})
    layers = (LayerSpec("blocks.0.", toy, ffn, norm("n1"), norm("n2")),
              LayerSpec("blocks.1.", attn, ffn, norm("n1"), norm("n2")),
              LayerSpec("blocks.2.", attn, ffn, norm("n1"), norm("n2")),
              LayerSpec("blocks.3.", turned, switch, norm("n1"), norm("n2")))
    # layer 0 runs twice (two states); layer 2 attends over the keys and values site 1 wrote; layer 3 has the toy
    # position encoding, the toy routed feed-forward and, with no window, pages of its own
    schedule = (Site(0), Site(1), Site(0), Site(2, cache_of=1), Site(3))
    return ModelSpec("ToyForCausalLM", H, raw["vocab"], layers, schedule, PartSpec("rmsnorm", {"eps": eps}),
                     embedding_name="tok.weight", final_norm_prefix="out_norm.", head_name="head.weight",
                     name_prefixes=("",))


def toy_plain(raw, W, tokens):
    """The toy model on a whole sequence, from the plain implementation's functions."""
    eps, H = raw["eps"], raw["width"]
    cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16, hidden_size=H, norm_eps=eps, rope_theta=1e4)
    h = W["tok.weight"][torch.tensor(tokens)]

    def toy(n, p):
        d = torch.sigmoid(W[p + "decay"])
        s, out = torch.zeros(H), []
        for t in range(n.shape[0]):
            s = d * s + n[t]
            out.append(s)
        return torch.stack(out)

    def ffn(h, p):
        return h + P.dense_mlp(P.rms_norm(h, W[p + "n2.weight"], eps), W, p)

    h = ffn(h + toy(P.rms_norm(h, W["blocks.0.n1.weight"], eps), "blocks.0."), "blocks.0.")
    # site 1: attention layer 1, windowed; its rotated keys and its values are what site 3 reads
    n1 = P.rms_norm(h, W["blocks.1.n1.weight"], eps)
    h = ffn(h + P.attention(n1, W, "blocks.1.", cfg, window=raw["window"]), "blocks.1.")
    h = ffn(h + toy(P.rms_norm(h, W["blocks.0.n1.weight"], eps), "blocks.0."), "blocks.0.")
    # site 3: layer 2's queries over site 1's keys and values
    n3 = P.rms_norm(h, W["blocks.2.n1.weight"], eps)
    mixed = {**{k.replace("blocks.1.", "x."): v for k, v in W.items() if k.startswith("blocks.1.")},
             "x.q_proj.weight": W["blocks.2.q_proj.weight"], "x.q_layernorm.weight": W["blocks.2.q_layernorm.weight"],
             "x.out_proj.weight": W["blocks.2.out_proj.weight"]}
    # keys and values come from site 1's input n1, queries from n3
    a = _cross_attention(n3, n1, mixed, cfg, raw["window"])
    h = ffn(h + a, "blocks.2.")
    # site 4: attention with pairs turned by position * 0.37, no window; then the switch feed-forward
    n4 = P.rms_norm(h, W["blocks.3.n1.weight"], eps)
    h = h + _turned_attention(n4, {k.replace("blocks.3.", "x."): v for k, v in W.items() if k.startswith("blocks.3.")}, cfg)
    n5 = P.rms_norm(h, W["blocks.3.n2.weight"], eps)
    choice = (n5 @ W["blocks.3.switch.weight"].T).argmax(-1)
    branch = torch.stack([torch.relu(n5[t] @ W[f"blocks.3.e{int(e)}.up.weight"].T) @ W[f"blocks.3.e{int(e)}.down.weight"].T
                          for t, e in enumerate(choice)])
    h = h + branch
    return P.rms_norm(h, W["out_norm.weight"], eps) @ W["head.weight"].T


def _turned_attention(n, W, cfg):
    T = n.shape[0]
    Hq, Hk, D, eps = 4, 2, 16, cfg["norm_eps"]
    q = P.rms_norm((n @ W["x.q_proj.weight"].T).view(T, Hq, D), W["x.q_layernorm.weight"], eps)
    k = P.rms_norm((n @ W["x.k_proj.weight"].T).view(T, Hk, D), W["x.k_layernorm.weight"], eps)
    v = (n @ W["x.v_proj.weight"].T).view(T, Hk, D)
    ang = torch.arange(T).float()[:, None, None] * 0.37

    def turn(t):
        a, b = t[..., 0::2], t[..., 1::2]
        out = torch.empty_like(t)
        out[..., 0::2], out[..., 1::2] = a * torch.cos(ang) - b * torch.sin(ang), a * torch.sin(ang) + b * torch.cos(ang)
        return out
    q, k = turn(q), turn(k)
    ks, vs = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    s = torch.einsum("thd,shd->hts", q, ks) * D ** -0.5
    i = torch.arange(T)
    a = torch.softmax(s.masked_fill((i[None, :] > i[:, None])[None], float("-inf")), -1)
    return torch.einsum("hts,shd->thd", a, vs).reshape(T, Hq * D) @ W["x.out_proj.weight"].T


def _cross_attention(nq, nkv, W, cfg, window):
    """P.attention with the queries computed from `nq` and the keys and values from `nkv` (same positions)."""
    T = nq.shape[0]
    Hq, Hk, D, eps = 4, 2, 16, cfg["norm_eps"]
    q = P.rms_norm((nq @ W["x.q_proj.weight"].T).view(T, Hq, D), W["x.q_layernorm.weight"], eps)
    k = P.rms_norm((nkv @ W["x.k_proj.weight"].T).view(T, Hk, D), W["x.k_layernorm.weight"], eps)
    v = (nkv @ W["x.v_proj.weight"].T).view(T, Hk, D)
    cos, sin = P.rotary_tables(torch.arange(T), D, cfg["rope_theta"], nq.dtype)
    cos, sin = cos[:, None, :], sin[:, None, :]
    q, k = q * cos + P.rotate_half(q) * sin, k * cos + P.rotate_half(k) * sin
    ks, vs = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    s = torch.einsum("thd,shd->hts", q, ks) * D ** -0.5
    i = torch.arange(T)
    hidden = (i[None, :] > i[:, None]) | (i[None, :] <= i[:, None] - window)
    a = torch.softmax(s.masked_fill(hidden[None], float("-inf")), -1)
    return torch.einsum("hts,shd->thd", a, vs).reshape(T, Hq * D) @ W["x.out_proj.weight"].T


def test_a_toy_architecture_registers_builds_and_steps(tmp_path):
    from tandemllm_b200.config import Architecture, register, unregister
    from tandemllm_b200.engine import Engine, EngineArgs, StepEntry
    from tandemllm_b200.parts import FEED_FORWARDS, MIXERS, POSITION_ENCODINGS, DecoderModel
    from tandemllm_b200.weights.random_init import random_tensor
    from tandemllm_b200.weights.safetensors_io import write_file
    register_toy()
    register_toy_switch_and_position()
    register(Architecture("toy", ("ToyForCausalLM",), ("toy",), lambda raw, folder, generation: toy_spec(raw)))
    try:
        raw = {"architectures": ["ToyForCausalLM"], "width": 48, "inner": 80, "vocab": 101, "eps": 1e-5, "window": 24}
        spec = toy_spec(raw)
        W = {s.name: random_tensor(s, 3, 0.15, 0.5, 0.1) for s in DecoderModel(spec).weight_specs()}
        (tmp_path / "config.json").write_text(json.dumps(raw))
        write_file(str(tmp_path / "model.safetensors"), W)
        eng = Engine.from_folder(str(tmp_path), EngineArgs(dtype="float32", max_len=512, parallel=2, kv_blocks=6))
        # site 1 owns the windowed group and site 3 borrows it; site 4, with no window, has pages of its own; the two
        # toy sites have a state slot each
        assert len(eng.cache.groups) == 2 and [g.need.window for g in eng.cache.groups] == [24, None]
        assert eng.cache.groups[0].sites == [1] and eng.cache.groups[1].sites == [4] and eng.cache._slot_sites == [0, 2]
        toks = torch.randint(0, 101, (90,), generator=torch.Generator().manual_seed(5)).tolist()
        want = toy_plain(raw, W, toks)
        eng.admit("t")
        outs, at = [], 0
        for n in (5, 2, 30, 1, 1, 20, 3, 28):
            outs.append(eng.step([StepEntry("t", toks[at:at + n], list(range(n)))]).cpu())
            at += n
        assert at == 90
        assert max_rel(torch.cat(outs), want) < 1e-4
        # 90 tokens went through 6 pages of 16 because the window gives pages back; the group without a window holds all
        assert eng.cache.groups[0].pool.used <= 3 and eng.cache.groups[1].pool.used == 6
        eng.release("t")
        assert eng.cache.groups[0].pool.free == 6 and eng.cache.groups[1].pool.free == 6
    finally:
        unregister("toy")
        MIXERS.pop("toy_decay", None)
        FEED_FORWARDS.pop("toy_switch", None)
        POSITION_ENCODINGS.pop("toy_pairs", None)


# ---- another architecture out of the product's own parts, with other constants: a GELU-gated dense feed-forward and
# experts routed by a softmax over all experts with a squared-ReLU gate, in both precisions through the fused kernels
def fused_toy_spec(raw):
    from tandemllm_b200.config import ModelSpec, PartSpec, Site
    from tandemllm_b200.config.spec import LayerSpec
    H, eps = raw["width"], raw["eps"]
    norm = lambda name: PartSpec("rmsnorm", {"eps": eps, "name": name})
    conv = PartSpec("short_conv", {"taps": 3, "names": {"in": "mix.in", "taps": "mix.taps", "out": "mix.out"}})
    attn = PartSpec("attention", {"num_heads": 4, "num_kv_heads": 1, "head_dim": 64, "qk_norm": PartSpec("rmsnorm", {"eps": eps}),
                                  "position": PartSpec("rope_neox", {"theta": 1e4, "rotary_dim": 64}), "window": None,
                                  "names": {"q": "att.q", "k": "att.k", "v": "att.v", "out": "att.o", "q_norm": "att.qn",
                                            "k_norm": "att.kn"}})
    dense = PartSpec("swiglu", {"intermediate_size": raw["inner"], "activation": "gelu",
                                "names": {"gate": "ff.g", "up": "ff.u", "down": "ff.d"}})
    routed = PartSpec("sigmoid_topk_experts", {"num_experts": raw["experts"], "top_k": 2, "intermediate_size": raw["expert_inner"],
                                               "expert_bias": False, "normalize": True, "scale": 1.0, "norm_floor": 0.0,
                                               "scoring": "softmax", "activation": "relu2",
                                               "names": {"router": "moe.router", "bias": "moe.bias", "experts": "moe.e",
                                                         "gate": "g", "up": "u", "down": "d"}})
    layers = (LayerSpec("b.0.", conv, dense, norm("n1"), norm("n2")), LayerSpec("b.1.", attn, routed, norm("n1"), norm("n2")),
              LayerSpec("b.2.", conv, routed, norm("n1"), norm("n2")))
    return ModelSpec("FusedToyForCausalLM", H, raw["vocab"], layers, tuple(Site(i) for i in range(3)),
                     PartSpec("rmsnorm", {"eps": eps}), embedding_name="tok.weight", final_norm_prefix="last.",
                     head_name="head.weight", name_prefixes=("",))


def fused_toy_plain(raw, W, tokens, forced=None):
    """(logits, routing margins) of the whole sequence in plain torch. `forced` {layer prefix: ids [T, 2]} replaces a
    routed layer's choice of experts (the weights are still this function's own)."""
    eps, H, E = raw["eps"], raw["width"], raw["experts"]
    cfg = dict(num_attention_heads=4, num_key_value_heads=1, head_dim=64, hidden_size=H, norm_eps=eps, rope_theta=1e4)
    h = W["tok.weight"][torch.tensor(tokens)]
    margins = []

    def conv(h, p):
        names = {"x.in_proj.weight": W[p + "mix.in.weight"], "x.conv.weight": W[p + "mix.taps.weight"],
                 "x.out_proj.weight": W[p + "mix.out.weight"]}
        return h + P.short_conv(P.rms_norm(h, W[p + "n1.weight"], eps), names, "x.", 3, False)

    def routed(h, p):
        n = P.rms_norm(h, W[p + "n2.weight"], eps)
        logits = n @ W[p + "moe.router.weight"].T
        score = torch.softmax(logits, -1)
        top = torch.sort(score, dim=-1, descending=True, stable=True)
        ordered = torch.sort(logits, dim=-1, descending=True).values
        margins.append(ordered[:, 1] - ordered[:, 2])          # how far, in logits, the choice is from another
        ids, w = top.indices[:, :2], top.values[:, :2]
        if forced is not None:
            ids = forced[p].long()
            w = torch.gather(score, 1, ids)
        w = w / w.sum(-1, keepdim=True)
        out = torch.zeros_like(n)
        for e in range(E):
            rows, slot = torch.where(ids == e)
            if rows.numel():
                q = f"{p}moe.e.{e}."
                y = (torch.relu(n[rows] @ W[q + "g.weight"].T) ** 2 * (n[rows] @ W[q + "u.weight"].T)) @ W[q + "d.weight"].T
                out.index_add_(0, rows, y * w[rows, slot, None])
        return h + out
    h = conv(h, "b.0.")
    n = P.rms_norm(h, W["b.0.n2.weight"], eps)
    h = h + (torch.nn.functional.gelu(n @ W["b.0.ff.g.weight"].T) * (n @ W["b.0.ff.u.weight"].T)) @ W["b.0.ff.d.weight"].T
    names = {"x." + k: W[f"b.1.att.{v}.weight"] for k, v in (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"),
                                                             ("out_proj.weight", "o"), ("q_layernorm.weight", "qn"),
                                                             ("k_layernorm.weight", "kn"))}
    h = h + P.attention(P.rms_norm(h, W["b.1.n1.weight"], eps), names, "x.", cfg)
    h = routed(h, "b.1.")
    h = routed(conv(h, "b.2."), "b.2.")
    return P.rms_norm(h, W["last.weight"], eps) @ W["head.weight"].T, torch.stack(margins).min(0).values


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_another_architecture_reuses_the_fused_kernels_with_its_own_activation_and_scoring(tmp_path, dtype, tol):
    """A routed model out of the product's own parts with a GELU-gated dense feed-forward and experts scored by a softmax
    over all experts with a squared-ReLU gate, registered from here. In bfloat16 it runs the fused tensor-core kernels (the
    persistent, the swapped and the register-only forms, decode steps from graphs). Every position is held to the plain
    implementation run with the engine's own choice of experts (read from a traced second run), so that a routing near tie
    is no excuse; in 32-bit the choice itself must be the plain implementation's."""
    from tandemllm_b200.config import Architecture, register, unregister
    from tandemllm_b200.engine import Engine, EngineArgs, StepEntry
    from tandemllm_b200.parts import DecoderModel
    from tandemllm_b200.weights.random_init import random_tensor
    from tandemllm_b200.weights.safetensors_io import write_file
    register(Architecture("fused_toy", ("FusedToyForCausalLM",), ("fused_toy",), lambda raw, folder, generation: fused_toy_spec(raw)))
    try:
        raw = {"architectures": ["FusedToyForCausalLM"], "width": 128, "inner": 192, "vocab": 200, "eps": 1e-5, "experts": 6,
               "expert_inner": 64}
        spec = fused_toy_spec(raw)
        W = {s.name: random_tensor(s, 5, 0.08, 0.5, 0.1).to(torch.bfloat16).float() for s in DecoderModel(spec).weight_specs()}
        (tmp_path / "config.json").write_text(json.dumps(raw))
        write_file(str(tmp_path / "model.safetensors"), {k: v.to(torch.bfloat16) if dtype == "bfloat16" else v for k, v in W.items()})
        toks = torch.randint(0, 200, (170,), generator=torch.Generator().manual_seed(8)).tolist()
        portions = (140, 9, 2) + (1,) * 19          # the persistent kernels, the swapped ones, the register-only ones, graphs

        def run(traced):
            eng = Engine.from_folder(str(tmp_path), EngineArgs(dtype=dtype, max_len=512, parallel=2, kv_blocks=32, graph=True))
            routes = {}
            if traced:
                eng.step_function.trace = {}
            eng.admit("t")
            outs, at = [], 0
            for n in portions:
                outs.append(eng.step([StepEntry("t", toks[at:at + n], list(range(n)))]).float().cpu())
                for prefix, ids in (eng.step_function.trace or {}).get("routes", []):
                    routes.setdefault(prefix, []).append(ids.cpu())
                at += n
            assert at == 170 and (traced or eng.step_function.graph_replays >= 10)
            eng.release("t")
            return torch.cat(outs), {p: torch.cat(v) for p, v in routes.items()}
        got, _ = run(False)
        again, routes = run(True)
        assert torch.equal(got, again), "a traced (eager) run gives the bits of the run with graphs"
        assert set(routes) == {"b.1.", "b.2."} and all(v.shape == (170, 2) for v in routes.values())
        plain_logits, margin = fused_toy_plain(raw, W, toks)
        if dtype == "float32":
            own = fused_toy_plain(raw, W, toks, forced=routes)[0]
            assert torch.equal(own, plain_logits) or float((own - plain_logits).abs().max()) < 1e-6, "32-bit: the same experts"
        want = fused_toy_plain(raw, W, toks, forced=routes)[0]
        err = (got - want).abs().amax(-1) / want.abs().amax(-1)
        assert float(err.max()) < tol, (float(err.max()), int(err.argmax()))
        # and the engine's own choice of experts is the plain implementation's at most positions
        differs = (got - plain_logits).abs().amax(-1) / plain_logits.abs().amax(-1) > tol
        assert int(differs.sum()) <= 40, int(differs.sum())
    finally:
        unregister("fused_toy")
