"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of LFM2-8B-A1B (24 layers, 18 conv and 6 attention, hidden 2048, 32/8 heads of
64, 32 experts top-4 of width 1792, dense width 7168, vocabulary 65536) with random bfloat16 weights, a batch of 8
requests at a context of 8192 tokens. A "step" is one decode step of the whole batch.

  value      decoded tokens a second, timed on the device with CUDA events over exactly K steps (the cache holds a
             synthetic context: random keys and values, since a step's time does not depend on their values)
  e2e        the same through the Python entry point (`Engine.run_step`): every step stages its tokens, positions and
             block tables in pinned host memory and copies them to the device, and reads the sampled tokens back
  prefill    one request of 2048 random tokens from an empty cache to its last logits; frac = flops / time / peak
  roofline   bytes the decode step has to read (every weight it uses once, counted from the experts the step really
             chose, plus the keys and values of the live requests) / time, against the measured copy bandwidth
  points     decoded tokens a second at batch 1 and 64

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else from an earlier measurement on the same
kind of machine (6.65 TB/s, 1.59 PFLOP/s). Every step reads far more than the 126 MB L2 holds (gigabytes of weights),
so nothing is flushed between steps; `config.l2` says so.
"""

from __future__ import annotations

import argparse
import json
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
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in raw:
                out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            return out
        except (ValueError, KeyError, OSError):
            pass
    return dict(FALLBACK_PEAKS)


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


def reference_arm() -> int:
    print(json.dumps({"impl": "reference", "unavailable":
                      "pip installs the reference's proxy, server and chatd packages only (pyproject.toml lists no "
                      "engine package): `import server.app` from baseline/_ref fails with No module named 'engine', "
                      "so no stock code path of the install generates tokens; its kernels also target sm_121a only"}))
    return 0


def decode_bytes(engine, batch: int, context: int, distinct_experts: list[int]) -> dict:
    """Bytes one decode step has to read: every weight it uses once, and the cache of the live requests."""
    model = engine.model
    elem = 2 if engine.args.dtype in ("bfloat16", "bf16") else 4
    H = model.hidden_size
    dense = experts = 0
    it = iter(distinct_experts)
    for site in model.spec.schedule:
        layer = model.layers[site.layer]
        m, f = layer.mixer, layer.feed_forward
        for name in ("w_qkv", "w_out", "w_in"):
            w = getattr(m, name, None)
            if w is not None:
                dense += w.numel() * elem
        if hasattr(f, "num_experts"):
            dense += f.w_router.numel() * 4
            per_expert = (f.w_gate_up.shape[1] * H + H * f.w_down.shape[2]) * elem
            experts += next(it) * per_expert
        else:
            dense += (f.w_gate_up.numel() + f.w_down.numel()) * elem
    head = model.head.numel() * elem
    kv = 0
    for g in engine.cache.groups:
        span = context if g.need.window is None else min(context, g.need.window)
        kv += len(g.sites) * 2 * g.need.kv_heads * g.need.head_dim * elem * span * batch
    return {"dense": dense, "experts": experts, "head": head, "kv": kv, "total": dense + experts + head + kv}


def prefill_flops(cfg, tokens: int) -> float:
    H, T = cfg.hidden_size, tokens
    per_token = 0
    for li in range(cfg.num_hidden_layers):
        if cfg.is_attention(li):
            per_token += 2 * H * (cfg.q_dim + 2 * cfg.kv_dim) + 2 * cfg.q_dim * H
        else:
            per_token += 2 * H * 3 * H + 2 * H * H
        if cfg.is_moe(li):
            per_token += 2 * H * cfg.num_experts + cfg.num_experts_per_tok * 6 * H * cfg.moe_intermediate_size
        else:
            per_token += 6 * H * cfg.intermediate_size
    attention = len(cfg.attention_layers) * 2 * T * T * cfg.q_dim        # causal: half of 4 T^2 Hq D
    return float(per_token) * T + attention + 2.0 * H * cfg.vocab_size


def mixed_serving(cfg, model_name: str, a) -> int:
    """Long-context mixed serving through the scheduler: what the line says. Not the headline; no roofline."""
    import math

    import torch

    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    requests, longest, new_tokens, budget_tokens = 64, 32768, 64, 262144
    engine = Engine.from_config(cfg, seed=0, args=EngineArgs(
        dtype=a.dtype, max_len=longest + new_tokens + 16, parallel=requests, block_size=16, kv_blocks=budget_tokens // 16,
        max_batched_tokens=2048, chunk_size=512, graph=a.graph == "on"))
    moe = [layer.feed_forward for layer in engine.model.layers if hasattr(layer.feed_forward, "num_experts")]
    for part in moe:
        part.load = torch.zeros(part.num_experts, dtype=torch.int64, device=engine.device)
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
    load = torch.stack([part.load for part in moe]).double()               # [layers, experts] pairs routed
    share = load / load.sum(1, keepdim=True)
    print(json.dumps({
        "scenario": "mixed serving", "model": model_name, "layers": cfg.num_hidden_layers, "requests": requests,
        "prompt_tokens": sum(lengths), "longest_prompt": max(lengths), "new_tokens_each": new_tokens,
        "cache_budget_tokens": budget_tokens, "page_tokens": 16, "portion": 512, "sampling": "greedy and temperature 0.8, alternating",
        "seconds": round(seconds, 2), "steps": steps, "tokens_per_s": round(st.rows / seconds, 1),
        "prompt_rows": st.prompt_rows, "decode_rows": st.decode_rows, "preemptions": st.preemptions,
        "pages_reused": engine.cache.groups[0].pool.reused, "graph_replays": engine.step_function.graph_replays,
        "expert_load": {"pairs_routed": int(load.sum()), "largest_share_of_a_layer": round(float(share.max()), 4),
                        "smallest_share_of_a_layer": round(float(share.min()), 4), "even_share": round(1.0 / load.shape[1], 4)},
        "dtype": "bf16" if a.dtype == "bfloat16" else "fp32", "data": "synthetic: random weights, uniform random token ids"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--sizes", default="8b", choices=("8b", "24b"),
                    help="layer sizes: LFM2-8B-A1B (the default and the headline) or the 24B-A2B class (40 layers, 64 experts)")
    ap.add_argument("--layers", type=int, default=0, help="run only the first N layers (the line names both numbers)")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--graph", default="on", choices=("on", "off"))
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (for profiling runs)")
    ap.add_argument("--only", choices=("prefill",), help="measure only this part and print it (a profiling aid)")
    ap.add_argument("--scenario", choices=("mixed",),
                    help="mixed: 64 requests with prompts of 128 to 32768 tokens (log-uniform) under a cache budget that makes "
                         "them queue, portions of 512 beside decode tokens, greedy and temperature 0.8 mixed, expert load "
                         "recorded; prints its own line (not the headline)")
    ap.add_argument("--chain", default="off", choices=("on", "off"),
                    help="programmatic dependent launch between the kernels (for comparison; ordinary launches by default)")
    ap.add_argument("--profile", action="store_true",
                    help="bracket the timed decode steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm()
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

    raw = dict(CONFIG_8B)
    model_name = "LFM2-8B-A1B layer sizes"
    if a.sizes == "24b":
        model_name = "LFM2.5-24B-A2B-class layer sizes"
        raw.update(num_hidden_layers=40, intermediate_size=11776, moe_intermediate_size=1536, num_experts=64,
                   layer_types=["full_attention" if i % 4 == 2 else "conv" for i in range(40)])
    layers_of_model = raw["num_hidden_layers"]
    a.layers = a.layers or layers_of_model
    if a.layers != layers_of_model:
        raw["layer_types"] = raw["layer_types"][:a.layers]
        raw["num_hidden_layers"] = a.layers
    cfg = Lfm2MoeConfig.from_dict(raw)
    if a.scenario == "mixed":
        return mixed_serving(cfg, model_name, a)
    pk = peaks()
    max_batch = 64 if not a.skip_points else a.batch
    room = a.context + a.steps + a.warmup + 80
    t0 = time.time()
    engine = Engine.from_config(cfg, seed=0, args=EngineArgs(
        dtype=a.dtype, max_len=room, parallel=max(max_batch, a.batch), block_size=16,
        max_batched_tokens=max(PREFILL_TOKENS, max_batch), chunk_size=PREFILL_TOKENS, graph=a.graph == "on"))
    torch.cuda.synchronize()
    load_s = time.time() - t0
    if a.chain == "on":
        from tandemllm_b200.kernels import tensorcore
        ops.core().tl_set_chained_launches(1)
        if a.dtype == "bfloat16":
            tensorcore.lib().tl_tc_set_chained_launches(1)
    for sc in engine.cache.site_cache:            # a synthetic context: random keys and values
        if hasattr(sc, "k"):
            sc.k.normal_(0, 0.5)
            sc.v.normal_(0, 0.5)
    g = torch.Generator().manual_seed(1)
    V = cfg.vocab_size
    greedy = SamplingParams(temperature=0.0, max_tokens=1 << 30, ignore_eos=True)

    def start(batch: int, context: int):
        return [engine.add_request_with_context(torch.randint(0, V, (context,), generator=g).tolist(),
                                                SamplingParams(**vars(greedy))) for _ in range(batch)]

    def finish(reqs):
        for r in reqs:
            engine.scheduler.abort(r)

    def device_decode(batch: int, context: int, steps: int, warmup: int) -> dict:
        """K decode steps timed on the device: given tokens in, argmax on the device, no host wait between steps."""
        reqs = start(batch, context)
        fn = engine.step_function
        fn.check_status = False
        toks = torch.randint(0, V, (steps + warmup, batch), generator=g).tolist()
        out = torch.empty(batch, dtype=torch.int32, device=engine.device)

        def one(i):
            entries = [StepEntry(r.request_id, [toks[i][j]], [0]) for j, r in enumerate(reqs)]
            ops.argmax(fn.run(entries), out)
        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        before = ops.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if a.profile:
            torch.cuda.profiler.start()
        e0.record()
        for i in range(warmup, warmup + steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
        if a.profile:
            torch.cuda.profiler.stop()
        ms = e0.elapsed_time(e1)
        launched = ops.launches - before
        fn.check_status = True
        fn.raise_on_fault()
        for r in reqs:                              # the scheduler's view of these requests is not used here
            r.num_computed = engine.cache.length_of(r.request_id)
        finish(reqs)
        return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launched}

    def e2e_decode(batch: int, context: int, steps: int, warmup: int) -> dict:
        """The same through Engine.run_step: host tokens in (pinned staging, one copy), sampled tokens back."""
        reqs = start(batch, context)
        for _ in range(warmup):
            engine.run_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t = time.perf_counter()
        e0.record()
        for _ in range(steps):
            engine.run_step()
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t
        ms = max(e0.elapsed_time(e1), wall * 1e3)
        pages = max(len(engine.cache.table(0, r.request_id)) for r in reqs) if engine.cache.groups else 0
        h2d = 4 * (3 * batch + (batch + 1) + batch + batch + len(engine.cache.groups) * batch * max(pages, 1))
        assert all(sum(t >= 0 for t in r.output) == warmup + steps for r in reqs)      # a pending token may follow
        finish(reqs)
        return {"tok_s": batch * steps / (ms / 1e3), "h2d": h2d, "d2h": 4 * batch}

    def distinct_experts(batch: int, context: int) -> list[int]:
        """Experts each MoE site really chose in one decode step of this batch."""
        reqs = start(batch, context)
        parts = [engine.model.layers[s.layer].feed_forward for s in engine.model.spec.schedule]
        parts = [p for p in parts if hasattr(p, "num_experts")]
        for p in parts:
            p.record_counts = True
        graph = engine.step_function.use_graphs if hasattr(engine.step_function, "use_graphs") else None
        if graph is not None:
            engine.step_function.use_graphs = False
        engine.run_step()
        out = [int((p.last_counts > 0).sum()) for p in parts]
        for p in parts:
            p.record_counts = False
        if graph is not None:
            engine.step_function.use_graphs = graph
        finish(reqs)
        return out

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
        flops = prefill_flops(cfg, tokens)
        return {"value": round(tokens / (ms / 1e3), 1), "tokens": tokens, "ms": round(ms, 3),
                "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4), "tflops": round(flops / ms / 1e9, 1)}

    if a.only == "prefill":          # a profiling aid: the prefill alone, its last repetition between profiler marks
        print(json.dumps({"prefill": prefill(PREFILL_TOKENS, reps=2)}))
        return 0
    clocks = Clocks().start()
    main_run = device_decode(a.batch, a.context, a.steps, a.warmup)
    e2e = e2e_decode(a.batch, a.context, a.steps, a.warmup)
    clock_summary = clocks.stop()
    experts_used = distinct_experts(a.batch, a.context)
    nbytes = decode_bytes(engine, a.batch, a.context, experts_used)
    achieved = nbytes["total"] / (main_run["ms_per_step"] / 1e3) / 1e9
    points = {}
    pre = None
    if not a.skip_points:
        few = max(16, a.steps // 2)
        points["decode_b1"] = round(device_decode(1, a.context, few, a.warmup)["tok_s"], 1)
        points["decode_b64"] = round(device_decode(64, a.context, few, a.warmup)["tok_s"], 1)
        pre = prefill(PREFILL_TOKENS)
    line = {
        "metric": f"decode tok/s at batch {a.batch}, context {a.context} ({model_name}, B200)",
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if a.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random weights N(0, 0.02), uniform random token ids, random keys and values as context",
        "impl": "ours",
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
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": nbytes["total"],
                     "of": pk["source"], "experts_read_per_layer": round(sum(experts_used) / max(len(experts_used), 1), 2)},
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
