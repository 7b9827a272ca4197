"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of LFM2-8B-A1B (24 layers, 18 conv and 6 attention, hidden 2048, 32/8 heads of
64, 32 experts top-4 of width 1792, dense width 7168, vocabulary 65536) with random bfloat16 weights, a batch of 8
requests at a context of 8192 tokens. A "step" is one decode step of the whole batch.

  value      decoded tokens a second, timed on the device with CUDA events: W warm-up steps, then `repeats` (3) regions
             of exactly K steps each, the median region reported (the cache holds a synthetic context: random keys and
             values, since a step's time does not depend on their values)
  e2e        the same through the Python entry point (`Engine.run_step`): every step stages its tokens, positions and
             block tables in pinned host memory and copies them to the device, and reads the sampled tokens back
  prefill    one request of 2048 random tokens from an empty cache to its last logits; frac = flops / time / the burst
             peak, frac_sustained against the sustained one
  roofline   bytes the decode step has to read (every weight it uses once, counted from the experts the step really
             chose, plus the keys and values of the live requests) / time, against the measured copy bandwidth
  points     decoded tokens a second at batch 1 and 64 with their roofline fractions, and the headline batch without
             CUDA graphs

Other modes: `--scenario mixed` (long-context serving through the scheduler, its own line; `--log FILE` writes the
engine's per-step records as JSON lines), `--profile-table` (one eager decode step and one prefill with every kernel
launch timed by CUDA events, summed by kernel family: milliseconds, the bytes or flops the family has to move or do,
and the fraction of the peak), `--impl reference` (the reference's own model code, see `reference_arm`).

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else from an earlier measurement on the same
kind of machine (6.65 TB/s, 1.59 PFLOP/s). Every step reads far more than the 126 MB L2 holds (gigabytes of weights),
so nothing is flushed between steps; `config.l2` says so.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYER_TYPES_8B = ["full_attention" if i in (2, 6, 10, 14, 18, 21) else "conv" for i in range(24)]
CONFIG_8B = dict(
    model_type="lfm2_moe", architectures=["Lfm2MoeForCausalLM"], vocab_size=65536, hidden_size=2048,
    intermediate_size=7168, moe_intermediate_size=1792, num_hidden_layers=24, num_attention_heads=32,
    num_key_value_heads=8, head_dim=64, norm_eps=1e-5, max_position_embeddings=128000, conv_bias=False, conv_L_cache=3,
    num_dense_layers=2, num_experts=32, num_experts_per_tok=4, use_expert_bias=True, routed_scaling_factor=1.0,
    norm_topk_prob=True, tie_word_embeddings=True, layer_types=LAYER_TYPES_8B,
    rope_parameters={"rope_type": "default", "rope_theta": 1000000.0}, eos_token_id=7, bos_token_id=1, pad_token_id=0)
CONTEXT = 8192
BATCH = 8
PREFILL_TOKENS = 2048
REPEATS = 3
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
REFERENCE_CHECKOUT = os.path.join(ROOT, "baseline", "_ref", "checkout")


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
            out["bf16_tflops_sustained"] = float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"]))
            return out
        except (ValueError, KeyError, OSError):
            pass
    return dict(FALLBACK_PEAKS)


def sized_config(sizes: str, layers: int) -> tuple[dict, str, int]:
    """(config.json dict, the model's name, layers of the whole model) for `--sizes` and `--layers`."""
    raw = dict(CONFIG_8B)
    name = "LFM2-8B-A1B layer sizes"
    if sizes == "24b":
        name = "LFM2.5-24B-A2B-class layer sizes"
        raw.update(num_hidden_layers=40, intermediate_size=11776, moe_intermediate_size=1536, num_experts=64,
                   layer_types=["full_attention" if i % 4 == 2 else "conv" for i in range(40)])
    whole = raw["num_hidden_layers"]
    layers = layers or whole
    if layers != whole:
        raw["layer_types"] = raw["layer_types"][:layers]
        raw["num_hidden_layers"] = layers
    return raw, name, whole


class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows, self.proc, self.thread = [], None, None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE, text=True)
        except OSError:
            return self
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for j, n in enumerate(names) if any(r[2 + j].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------ the reference arm
def reference_arm(a) -> int:
    """The reference's own model code on the same sizes, weights of the same distribution and the same synthetic
    context: `Lfm2MoeRef` (engine/models/lfm2_moe/ref.py), the plain-torch model that the reference checks its engines
    against, in bfloat16 on cuda:0 (on the CPU where there is no GPU), driven the way its `generate_greedy`
    (engine/spec.py:150-199) drives a model: one sequence's token in, argmax out, per step. A batch of B is B of its
    sequence states decoded one after another, since that model has no batched step.

    Why this and not its fast engine: `pip install` of the reference gives the `proxy`, `server` and `chatd` packages
    only (its pyproject.toml lists no `engine` package), and the fast engine (engine/models/lfm2_moe/engine.py) needs
    the EXL3 and row kernels built for sm_121a and a GB10 / Ada adapter (tools/gpu/__init__.py:20-27). The `engine`
    package is therefore taken as it is from a checkout: `cp -r <checkout>/engine baseline/_ref/checkout/engine`
    (or `--reference <checkout>`). Without it this arm prints its `unavailable` line."""
    src = a.reference or REFERENCE_CHECKOUT
    if not os.path.isfile(os.path.join(src, "engine", "models", "lfm2_moe", "ref.py")):
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip installs the reference's proxy, server and chatd packages only (pyproject.toml lists no "
                          f"engine package), and no checkout of its engine package was found at {src} "
                          "(cp -r <checkout>/engine baseline/_ref/checkout/engine, or --reference <checkout>)"}))
        return 0
    if a.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference's model code runs one sequence on one device; "
                          f"--gpus {a.gpus} has no meaning for it", "n_gpus": a.gpus}))
        return 0
    sys.path.insert(0, src)
    import torch
    from engine.models.lfm2_moe.config import config_from_dict
    from engine.models.lfm2_moe.ref import Lfm2MoeRef

    raw, model_name, whole = sized_config(a.sizes, a.layers)
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda:0" if cuda else "cpu")
    if not cuda and not a.layers:
        raw, model_name, whole = sized_config(a.sizes, 4)          # the CPU: a few layers, and the line says so
    cfg = config_from_dict(raw, "bench")
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    g = torch.Generator(device=dev).manual_seed(0)

    def r(*shape, std=0.02, dt=dtype):
        return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std).to(dt)

    H, V, D = cfg.hidden_size, cfg.vocab_size, cfg.head_dim
    W = {"embed_tokens.weight": r(V, H), "embedding_norm.weight": torch.ones(H, device=dev, dtype=dtype)}
    for li in range(cfg.num_hidden_layers):
        p = f"layers.{li}."
        W[p + "operator_norm.weight"] = torch.ones(H, device=dev, dtype=dtype)
        W[p + "ffn_norm.weight"] = torch.ones(H, device=dev, dtype=dtype)
        if cfg.is_attention(li):
            q = p + "self_attn."
            W[q + "q_proj.weight"] = r(cfg.num_attention_heads * D, H)
            W[q + "k_proj.weight"] = r(cfg.num_key_value_heads * D, H)
            W[q + "v_proj.weight"] = r(cfg.num_key_value_heads * D, H)
            W[q + "out_proj.weight"] = r(H, cfg.num_attention_heads * D)
            W[q + "q_layernorm.weight"] = torch.ones(D, device=dev, dtype=dtype)
            W[q + "k_layernorm.weight"] = torch.ones(D, device=dev, dtype=dtype)
        else:
            W[p + "conv.in_proj.weight"] = r(3 * H, H)
            W[p + "conv.conv.weight"] = r(H, 1, cfg.conv_L_cache)
            W[p + "conv.out_proj.weight"] = r(H, H)
        f = p + "feed_forward."
        if cfg.is_moe(li):
            W[f + "gate.weight"] = r(cfg.num_experts, H)
            W[f + "expert_bias"] = r(cfg.num_experts, std=0.1, dt=torch.float32)
            for e in range(cfg.num_experts):
                W[f + f"experts.{e}.w1.weight"] = r(cfg.moe_intermediate_size, H)
                W[f + f"experts.{e}.w3.weight"] = r(cfg.moe_intermediate_size, H)
                W[f + f"experts.{e}.w2.weight"] = r(H, cfg.moe_intermediate_size)
        else:
            W[f + "w1.weight"] = r(cfg.intermediate_size, H)
            W[f + "w3.weight"] = r(cfg.intermediate_size, H)
            W[f + "w2.weight"] = r(H, cfg.intermediate_size)
    ref = Lfm2MoeRef(cfg, W, dtype=dtype, device=dev)
    steps, warmup = a.steps, max(3, a.warmup)
    hg = torch.Generator().manual_seed(1)

    def sync():
        if cuda:
            torch.cuda.synchronize()

    def decode(batch: int, context: int, steps: int, warmup: int) -> dict:
        states = []
        for _ in range(batch):
            st = ref.new_state(context + REPEATS * steps + warmup + 8)
            for li in st.k:                                   # a synthetic context, as in the other arm
                st.k[li][:, :context - 1].normal_(0, 0.5)
                st.v[li][:, :context - 1].normal_(0, 0.5)
            st.length = context - 1
            states.append(st)
        toks = torch.randint(0, V, (batch,), generator=hg).tolist()

        def one():
            for j, st in enumerate(states):
                toks[j] = int(ref.decode(toks[j], st)[-1].argmax())      # host token in, host token out
        for _ in range(warmup):
            one()
        sync()
        regions = []
        for _ in range(REPEATS):
            t0 = time.perf_counter()
            for _ in range(steps):
                one()
            sync()
            regions.append((time.perf_counter() - t0) * 1e3)
        ms = statistics.median(regions)
        del states
        return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "regions_ms": regions}

    clocks = Clocks().start()
    main_run = decode(a.batch, a.context, steps, warmup)
    clock_summary = clocks.stop()
    points = {}
    pre = None
    if not a.skip_points:
        points["decode_b1"] = round(decode(1, a.context, max(4, steps // 4), 3)["tok_s"], 1)
        st = ref.new_state(PREFILL_TOKENS + 8)
        prompt = torch.randint(0, V, (PREFILL_TOKENS,), generator=hg)
        times = []
        for i in range(2):
            st.reset_inplace()
            sync()
            t0 = time.perf_counter()
            ref.prefill(prompt, st)
            sync()
            times.append((time.perf_counter() - t0) * 1e3)
        pre = {"value": round(PREFILL_TOKENS / (min(times) / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(min(times), 1)}
    line = {
        "metric": f"decode tok/s at batch {a.batch}, context {a.context} ({model_name}, B200)",
        "value": round(main_run["tok_s"], 2), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if a.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random weights N(0, 0.02), uniform random token ids, random keys and values as context",
        "impl": "reference",
        "what": "the reference's Lfm2MoeRef (plain torch, its own unmodified file) on " + str(dev) + ", one sequence state a "
                "request, decoded one after another; its fast engine needs sm_121a kernels",
        "config": {"model": model_name, "layers": cfg.num_hidden_layers, "layers_of_model": whole,
                   "hidden": H, "experts": cfg.num_experts, "vocab": V, "global_batch": a.batch, "seq_len": a.context,
                   "parallelism": "none (1 GPU)", "device": str(dev)},
        "e2e": {"value": round(main_run["tok_s"], 2), "unit": "tok/s", "h2d_bytes_per_step": 8 * a.batch,
                "d2h_bytes_per_step": 8 * a.batch, "note": "the timed loop is host tokens in, host tokens out"},
        "gpu_launches": None, "repeats": REPEATS, "clocks": clock_summary,
    }
    if pre is not None:
        line["prefill"] = pre
        line["points"] = points
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------ helpers of our arm
def prefill_flops(cfg, tokens: int) -> dict:
    """Flops of a prompt of `tokens` tokens by family (multiply-adds times two; the head for the last row only)."""
    H, T = cfg.hidden_size, tokens
    dense = experts = router = 0
    for li in range(cfg.num_hidden_layers):
        if cfg.is_attention(li):
            dense += 2 * H * (cfg.q_dim + 2 * cfg.kv_dim) + 2 * cfg.q_dim * H
        else:
            dense += 2 * H * 3 * H + 2 * H * H
        if cfg.is_moe(li):
            router += 2 * H * cfg.num_experts
            experts += cfg.num_experts_per_tok * 6 * H * cfg.moe_intermediate_size
        else:
            dense += 6 * H * cfg.intermediate_size
    attention = len(cfg.attention_layers) * 2 * T * T * cfg.q_dim        # causal: half of 4 T^2 Hq D
    out = {"dense": float(dense) * T + 2.0 * H * cfg.vocab_size, "experts": float(experts) * T, "router": float(router) * T,
           "attention": float(attention)}
    out["total"] = sum(out.values())
    return out


def start_with_context(engine, prompt: list[int], params):
    """A running request whose prompt, except its last token, counts as already computed: its pages are reserved and
    hold whatever they held (the caller fills the cache tensors with random values), so a decode step at a long
    context is timed without running the prompt. The text it generates means nothing."""
    req = engine.add_request(prompt, params)
    sch, cache = engine.scheduler, engine.cache
    sch.waiting.remove(req)
    cache.admit(req.request_id)
    n = len(req.prompt) - 1
    cache.reserve(req.request_id, n)
    cache.advance(req.request_id, n)
    req.num_computed = n
    req.state = "running"
    sch.running.append(req)
    return req


class LaunchTimer:
    """Times every launcher call of the package's two libraries with a pair of CUDA events (a launcher is one kernel,
    sometimes two), so that a step's time can be summed by kernel family without a profiler. The events themselves
    cost a little: compare shares, and the sum with the step's own time."""

    def __init__(self):
        import torch
        from tandemllm_b200.kernels import ops, tensorcore
        self.torch = torch
        self.libs = [ops.core(), tensorcore.lib()]
        self.saved = []
        self.calls = []

    @staticmethod
    def family(name: str, args: tuple) -> str:
        if name == "tl_gemm_tc":
            grouped, swiglu, persistent = bool(args[17]), bool(args[15]), not args[13] and args[14] == 256
            if grouped:
                return "experts gate/up + SwiGLU (tcgen05)" if swiglu else "experts down (tcgen05)"
            return "dense products (tcgen05" + (", persistent)" if persistent else ", swapped)")
        if name == "tl_gemm_tc_pair":            # args: ..., gated at 13, ..., tile_group at 15
            grouped, gated = bool(args[15]), bool(args[13])
            if grouped:
                return "experts gate/up + SwiGLU (tcgen05)" if gated else "experts down (tcgen05)"
            return "dense products (tcgen05, pairs of SMs)"
        if name == "tl_gemm_skinny_grouped":
            return "experts gate/up + SwiGLU (register-only)" if args[11] else "experts down (register-only)"
        return {"tl_gemm_skinny_mma": "dense products (register-only)", "tl_gemm_skinny_conv": "in-projection + short conv",
                "tl_add_rmsnorm": "residual add + norm (+ router, + deferred sums)", "tl_paged_attention_mma": "attention", "tl_paged_attention_tc": "attention",
                "tl_paged_attention_split": "attention", "tl_paged_attention_simt": "attention",
                "tl_attention_join": "attention join", "tl_qk_prepare": "q/k norm + rotary + cache write",
                "tl_moe_plan": "routing plan", "tl_gather_rows": "rows into expert order", "tl_short_conv": "short conv",
                "tl_short_conv_decode": "short conv", "tl_short_conv_state": "short conv", "tl_embed_rows": "embedding",
                "tl_gemm_simt": "32-bit products", "tl_gemm_simt_grouped": "32-bit expert products",
                "tl_gated_mul": "gate activation", "tl_argmax": "argmax", "tl_sample": "sampling",
                "tl_router_topk": "router top-k", "tl_moe_combine": "expert combine", "tl_kv_store": "cache write"}.get(name, name)

    def __enter__(self):
        torch = self.torch
        for lib in self.libs:
            for name in [n for n in dir(lib) if n.startswith("tl_")] + list(getattr(lib, "__dict__", {})):
                fn = getattr(lib, name, None)
                if not name.startswith("tl_") or fn is None or getattr(fn, "restype", None) is None or \
                        not getattr(fn, "argtypes", None) or any((lib, name) == s[:2] for s in self.saved):
                    continue
                if len(fn.argtypes) >= 4 and fn.argtypes[-1] is ctypes.c_void_p:      # a launcher: its last argument is the stream
                    def wrapped(*args, _fn=fn, _name=name):
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                        code = _fn(*args)
                        e1.record()
                        self.calls.append((self.family(_name, args), e0, e1))
                        return code
                    self.saved.append((lib, name, fn))
                    setattr(lib, name, wrapped)
        return self

    def __exit__(self, *exc):
        for lib, name, fn in self.saved:
            setattr(lib, name, fn)
        self.saved = []

    def table(self) -> dict:
        self.torch.cuda.synchronize()
        out: dict = {}
        for fam, e0, e1 in self.calls:
            row = out.setdefault(fam, {"launches": 0, "ms": 0.0})
            row["launches"] += 1
            row["ms"] += e0.elapsed_time(e1)
        self.calls = []
        return out


def mixed_serving(cfg, model_name: str, a) -> int:
    """Long-context mixed serving through the scheduler: what the line says. Not the headline; no roofline.
    With `--check` the sizes shrink to what the plain implementation can follow and every generated token of the
    greedy requests is compared with it."""
    import torch

    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    requests, longest, new_tokens, budget_tokens = a.requests, a.longest, a.new_tokens, a.budget_tokens
    engine = Engine.from_config(cfg, seed=0, args=EngineArgs(
        dtype=a.dtype, max_len=longest + new_tokens + 16, parallel=requests, block_size=16, kv_blocks=budget_tokens // 16,
        max_batched_tokens=2048, chunk_size=512, graph=a.graph == "on", log=a.log, record_routing=True))
    g = torch.Generator().manual_seed(5)
    lengths = [int(math.exp(math.log(128) + float(torch.rand(1, generator=g)) * math.log(longest / 128))) for _ in range(requests)]
    reqs = []
    for i, n in enumerate(lengths):
        sp = SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True) if i % 2 == 0 else \
            SamplingParams(temperature=0.8, top_k=50, top_p=0.95, seed=100 + i, max_tokens=new_tokens, ignore_eos=True)
        reqs.append(engine.add_request(torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(), sp))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    steps = 0
    while engine.scheduler.has_unfinished():
        engine.run_step()
        steps += 1
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    st = engine.scheduler.stats
    assert all(len(r.output) == new_tokens and min(r.output) >= 0 for r in reqs)
    engine.cache.check()
    records = list(engine.records)
    load = sum(r["routed"] for r in records if "routed" in r)               # pairs routed to each expert, all layers in a row
    per_layer = load.reshape(-1, cfg.num_experts).astype("float64")
    share = per_layer / per_layer.sum(1, keepdims=True)
    touched = [sum(r["experts_touched"]) / max(len(r["experts_touched"]), 1) for r in records if "experts_touched" in r]
    print(json.dumps({
        "scenario": "mixed serving", "model": model_name, "layers": cfg.num_hidden_layers, "requests": requests,
        "prompt_tokens": sum(lengths), "longest_prompt": max(lengths), "new_tokens_each": new_tokens,
        "cache_budget_tokens": budget_tokens, "page_tokens": 16, "portion": 512, "sampling": "greedy and temperature 0.8, alternating",
        "seconds": round(seconds, 2), "steps": steps, "tokens_per_s": round(st.rows / seconds, 1),
        "prompt_rows": st.prompt_rows, "decode_rows": st.decode_rows, "preemptions": st.preemptions,
        "pages_reused": engine.cache.groups[0].pool.reused, "graph_replays": engine.step_function.graph_replays,
        "graphs_kept": len(engine.step_function._graphs), "graphs_dropped": engine.step_function.graphs_dropped,
        "expert_load": {"recorded": "per step (the engine's step records; --log FILE writes them)",
                        "pairs_routed": int(load.sum()), "largest_share_of_a_layer": round(float(share.max()), 4),
                        "smallest_share_of_a_layer": round(float(share.min()), 4), "even_share": round(1.0 / cfg.num_experts, 4),
                        "experts_touched_a_layer_per_step": {"min": round(min(touched), 2), "median": round(statistics.median(touched), 2),
                                                             "max": round(max(touched), 2)}},
        "dtype": "bf16" if a.dtype == "bfloat16" else "fp32", "data": "synthetic: random weights, uniform random token ids"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--reference", help="a checkout of the reference project (default: baseline/_ref/checkout)")
    ap.add_argument("--sizes", default="8b", choices=("8b", "24b"),
                    help="layer sizes: LFM2-8B-A1B (the default and the headline) or the 24B-A2B class (40 layers, 64 experts)")
    ap.add_argument("--layers", type=int, default=0, help="run only the first N layers (the line names both numbers)")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--graph", default="on", choices=("on", "off"))
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (for profiling runs)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="with --only prefill or --profile-table: a prompt of this many tokens in one step (the headline line keeps 2048)")
    ap.add_argument("--only", choices=("prefill",), help="measure only this part and print it (a profiling aid)")
    ap.add_argument("--scenario", choices=("mixed",),
                    help="mixed: 64 requests with prompts of 128 to 32768 tokens (log-uniform) under a cache budget that makes "
                         "them queue, portions of 512 beside decode tokens, greedy and temperature 0.8 mixed, expert load "
                         "recorded per step; prints its own line (not the headline)")
    ap.add_argument("--requests", type=int, default=64, help="mixed scenario: requests")
    ap.add_argument("--longest", type=int, default=32768, help="mixed scenario: longest prompt")
    ap.add_argument("--new-tokens", type=int, default=64, help="mixed scenario: tokens generated per request")
    ap.add_argument("--budget-tokens", type=int, default=262144, help="mixed scenario: tokens the cache holds")
    ap.add_argument("--log", help="mixed scenario: write the engine's per-step records here as JSON lines")
    ap.add_argument("--profile-table", action="store_true",
                    help="time every kernel launch of one eager decode step and one prefill with CUDA events and print "
                         "milliseconds, bytes or flops and the fraction of the peak by kernel family")
    ap.add_argument("--chain", default="off", choices=("on", "off"),
                    help="programmatic dependent launch between the kernels (for comparison; ordinary launches by default)")
    ap.add_argument("--profile", action="store_true",
                    help="bracket the timed decode steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {a.gpus} is not implemented", "n_gpus": a.gpus}))
        return 2
    if a.warmup < 3:
        a.warmup = 3

    import torch

    from tandemllm_b200.config import Lfm2MoeConfig
    from tandemllm_b200.engine import Engine, EngineArgs, StepEntry
    from tandemllm_b200.kernels import ops
    from tandemllm_b200.sampling import SamplingParams

    raw, model_name, layers_of_model = sized_config(a.sizes, a.layers)
    a.layers = raw["num_hidden_layers"]
    cfg = Lfm2MoeConfig.from_dict(raw)
    if a.scenario == "mixed":
        return mixed_serving(cfg, model_name, a)
    pk = peaks()
    bf16 = a.dtype == "bfloat16"
    max_batch = 64 if not a.skip_points else a.batch
    only_tokens = a.prefill_tokens if a.only == "prefill" or a.profile_table else PREFILL_TOKENS
    room = max(a.context, only_tokens) + REPEATS * a.steps + a.warmup + 80
    t0 = time.time()
    engine = Engine.from_config(cfg, seed=0, args=EngineArgs(
        dtype=a.dtype, max_len=room, parallel=max(max_batch, a.batch), block_size=16,
        max_batched_tokens=max(only_tokens, max_batch), chunk_size=only_tokens, graph=a.graph == "on"))
    torch.cuda.synchronize()
    load_s = time.time() - t0
    if a.chain == "on":
        from tandemllm_b200.kernels import tensorcore
        ops.core().tl_set_chained_launches(1)
        if bf16:
            tensorcore.lib().tl_tc_set_chained_launches(1)
    for sc in engine.cache.site_cache:            # a synthetic context: random keys and values
        if hasattr(sc, "k"):
            sc.k.normal_(0, 0.5)
            sc.v.normal_(0, 0.5)
    g = torch.Generator().manual_seed(1)
    V = cfg.vocab_size
    greedy = SamplingParams(temperature=0.0, max_tokens=1 << 30, ignore_eos=True)

    def start(batch: int, context: int):
        return [start_with_context(engine, torch.randint(0, V, (context,), generator=g).tolist(),
                                   SamplingParams(**vars(greedy))) for _ in range(batch)]

    def finish(reqs):
        for r in reqs:
            engine.scheduler.abort(r)

    def device_decode(batch: int, context: int, steps: int, warmup: int, repeats: int = REPEATS, graphs: bool | None = None) -> dict:
        """`repeats` regions of exactly `steps` decode steps, each timed on the device: given tokens in, argmax on the
        device, no host wait between steps. The median region is reported."""
        reqs = start(batch, context)
        fn = engine.step_function
        fn.check_status = False
        kept = fn.use_graphs
        if graphs is not None:
            fn.use_graphs = graphs and kept
        toks = torch.randint(0, V, (repeats * steps + warmup, batch), generator=g).tolist()
        out = torch.empty(batch, dtype=torch.int32, device=engine.device)

        def one(i):
            entries = [StepEntry(r.request_id, [toks[i][j]], [0]) for j, r in enumerate(reqs)]
            ops.argmax(fn.run(entries), out)
        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        regions, launched = [], 0
        for rep in range(repeats):
            before = ops.launches
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if a.profile and rep == 0:
                torch.cuda.profiler.start()
            e0.record()
            for i in range(warmup + rep * steps, warmup + (rep + 1) * steps):
                one(i)
            e1.record()
            torch.cuda.synchronize()
            if a.profile and rep == 0:
                torch.cuda.profiler.stop()
            regions.append(e0.elapsed_time(e1))
            launched = ops.launches - before
        ms = statistics.median(regions)
        fn.check_status = True
        fn.use_graphs = kept
        fn.raise_on_fault()
        for r in reqs:                              # the scheduler's view of these requests is not used here
            r.num_computed = engine.cache.length_of(r.request_id)
        finish(reqs)
        return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launched,
                "regions_ms": [round(x, 3) for x in regions]}

    def e2e_decode(batch: int, context: int, steps: int, warmup: int) -> dict:
        """The same through Engine.run_step: host tokens in (pinned staging, one copy), sampled tokens back."""
        reqs = start(batch, context)
        for _ in range(warmup):
            engine.run_step()
        torch.cuda.synchronize()
        regions = []
        for _ in range(REPEATS):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t = time.perf_counter()
            e0.record()
            for _ in range(steps):
                engine.run_step()
            e1.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t
            regions.append(max(e0.elapsed_time(e1), wall * 1e3))
        ms = statistics.median(regions)
        pages = max(len(engine.cache.table(0, r.request_id)) for r in reqs) if engine.cache.groups else 0
        h2d = 4 * (3 * batch + (batch + 1) + batch + batch + len(engine.cache.groups) * batch * max(pages, 1))
        assert all(sum(t >= 0 for t in r.output) == warmup + REPEATS * steps for r in reqs)      # a pending token may follow
        finish(reqs)
        return {"tok_s": batch * steps / (ms / 1e3), "h2d": h2d, "d2h": 4 * batch}

    def distinct_experts(batch: int, context: int) -> list[int]:
        """Experts each routed site really read in one decode step of this batch (from the engine's step record)."""
        engine.set_routing_record(True)
        reqs = start(batch, context)
        engine.run_step()
        out = list(engine.last_record.get("experts_touched", []))
        finish(reqs)
        engine.set_routing_record(False)
        return out

    def roofline(batch: int, context: int, ms_per_step: float) -> dict:
        experts_used = distinct_experts(batch, context)
        nbytes = engine.decode_bytes(batch, context, experts_used)
        achieved = nbytes["total"] / (ms_per_step / 1e3) / 1e9
        return {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": nbytes["total"], "of": pk["source"],
                "experts_read_per_layer": round(sum(experts_used) / max(len(experts_used), 1), 2), "parts": nbytes}

    def prefill(tokens: int, reps: int = 3) -> dict:
        times = []
        for i in range(reps + 1):
            engine.admit("prefill")
            prompt = torch.randint(0, V, (tokens,), generator=g).tolist()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if a.profile and i == reps:
                torch.cuda.profiler.start()
            e0.record()
            engine.step([StepEntry("prefill", prompt, [tokens - 1])])
            e1.record()
            torch.cuda.synchronize()
            if a.profile and i == reps:
                torch.cuda.profiler.stop()
            engine.release("prefill")
            if i:
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        flops = prefill_flops(cfg, tokens)["total"]
        peak = pk["bf16_tflops"] if bf16 else None
        out = {"value": round(tokens / (ms / 1e3), 1), "tokens": tokens, "ms": round(ms, 3),
               "tflops": round(flops / ms / 1e9, 1), "repeats": reps}
        if peak:
            out["frac"] = round(flops / (ms / 1e3) / (peak * 1e12), 4)
            out["frac_sustained"] = round(flops / (ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
        else:
            out["frac"] = None            # the 32-bit path runs on the CUDA cores: no tensor-core peak applies
        return out

    def profile_table() -> int:
        """One eager decode step and one prefill with every launch timed: ms, bytes or flops and fraction by family."""
        fn = engine.step_function
        fn.use_graphs = False
        reqs = start(a.batch, a.context)
        toks = torch.randint(0, V, (8, a.batch), generator=g).tolist()
        out = torch.empty(a.batch, dtype=torch.int32, device=engine.device)

        def one(i):
            ops.argmax(fn.run([StepEntry(r.request_id, [toks[i][j]], [0]) for j, r in enumerate(reqs)]), out)
        for i in range(3):
            one(i)
        torch.cuda.synchronize()
        timer = LaunchTimer()
        with timer:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            one(3)
            e1.record()
            decode = timer.table()
            eager_ms = e0.elapsed_time(e1)
        for r in reqs:
            r.num_computed = engine.cache.length_of(r.request_id)
        finish(reqs)
        nbytes = roofline(a.batch, a.context, 1.0)["parts"]
        H = cfg.hidden_size
        family_bytes = {"experts": nbytes["experts"], "dense": nbytes["dense"] + nbytes["head"], "attention": nbytes["kv"]}
        sums = {"experts": 0.0, "dense": 0.0, "attention": 0.0}
        for fam, row in decode.items():
            key = "experts" if fam.startswith("experts") else "dense" if fam.startswith(("dense", "in-projection")) else \
                "attention" if fam == "attention" else None
            if key:
                sums[key] += row["ms"]
            row["ms"] = round(row["ms"], 4)
        for key, ms in sums.items():
            if ms:
                decode[f"= {key}, all forms"] = {"ms": round(ms, 4), "bytes": family_bytes[key],
                                                 "GBps": round(family_bytes[key] / ms / 1e6, 1),
                                                 "frac_hbm": round(family_bytes[key] / ms / 1e6 / pk["hbm_gbs"], 4)}
        total = sum(r["ms"] for k, r in decode.items() if not k.startswith("="))
        engine.admit("prefill")
        prompt = torch.randint(0, V, (only_tokens,), generator=g).tolist()
        engine.step([StepEntry("prefill", prompt, [only_tokens - 1])])
        engine.release("prefill")
        engine.admit("prefill")
        with timer:
            engine.step([StepEntry("prefill", prompt, [only_tokens - 1])])
            pre = timer.table()
        engine.release("prefill")
        flops = prefill_flops(cfg, only_tokens)
        psums = {"experts": 0.0, "dense": 0.0, "attention": 0.0}
        for fam, row in pre.items():
            key = "experts" if fam.startswith("experts") else "dense" if fam.startswith("dense") else \
                "attention" if fam == "attention" else None
            if key:
                psums[key] += row["ms"]
            row["ms"] = round(row["ms"], 4)
        ptotal = sum(r["ms"] for r in pre.values())
        for key, ms in psums.items():
            if ms:
                pre[f"= {key}, all forms"] = {"ms": round(ms, 4), "flops": flops[key], "TFLOPs": round(flops[key] / ms / 1e9, 1),
                                              "frac_bf16_burst": round(flops[key] / ms / 1e9 / pk["bf16_tflops"], 4)}
        print(json.dumps({"profile_table": {"model": model_name, "layers": a.layers, "dtype": a.dtype, "batch": a.batch,
                                            "context": a.context, "peaks": pk,
                                            "decode_step": {"eager_ms": round(eager_ms, 4), "sum_of_launches_ms": round(total, 4),
                                                            "families": decode},
                                            "prefill": {"tokens": only_tokens, "sum_of_launches_ms": round(ptotal, 4),
                                                        "families": pre}}}))
        return 0

    if a.only == "prefill":          # a profiling aid: the prefill alone, its last repetition between profiler marks
        print(json.dumps({"prefill": prefill(only_tokens, reps=2)}))
        return 0
    if a.profile_table:
        return profile_table()
    clocks = Clocks().start()
    main_run = device_decode(a.batch, a.context, a.steps, a.warmup)
    e2e = e2e_decode(a.batch, a.context, a.steps, a.warmup)
    clock_summary = clocks.stop()
    roof = roofline(a.batch, a.context, main_run["ms_per_step"])
    roof.pop("parts")
    points = {}
    pre = None
    if not a.skip_points:
        few = max(16, a.steps // 2)
        for b in (1, 64):
            run = device_decode(b, a.context, few, a.warmup)
            points[f"decode_b{b}"] = round(run["tok_s"], 1)
            points[f"decode_b{b}_frac"] = roofline(b, a.context, run["ms_per_step"])["frac"]
        if a.graph == "on":
            points[f"decode_b{a.batch}_eager"] = round(device_decode(a.batch, a.context, few, a.warmup, graphs=False)["tok_s"], 1)
        pre = prefill(PREFILL_TOKENS)
    line = {
        "metric": f"decode tok/s at batch {a.batch}, context {a.context} ({model_name}, B200)",
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if bf16 else "fp32",
        "data": "synthetic: random weights N(0, 0.02), uniform random token ids, random keys and values as context",
        "impl": "ours", "repeats": REPEATS, "regions_ms": main_run["regions_ms"],
        "config": {"model": model_name, "layers": a.layers, "layers_of_model": layers_of_model,
                   "conv_layers": len(cfg.conv_layers), "attention_layers": len(cfg.attention_layers),
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "dense_ffn": cfg.intermediate_size, "experts": cfg.num_experts,
                   "top_k": cfg.num_experts_per_tok, "expert_ffn": cfg.moe_intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": a.batch, "seq_len": a.context, "parallelism": "none (1 GPU)", "page_tokens": 16,
                   "graph": a.graph, "l2": "inputs>L2 (a step reads GBs of weights)"},
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": main_run["launches"],
        "roofline": roof,
        "clocks": clock_summary,
        "load_s": round(load_s, 1),
    }
    if pre is not None:
        line["prefill"] = pre
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
