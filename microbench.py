"""Single kernels on small cases, timed with CUDA events: the commands behind the summaries under `profiles/`.

    python microbench.py expert_gemm --tokens 8
    python microbench.py dense_gemm --rows 8 --n 6144 --k 2048
    python microbench.py dense_gemm --rows 2048 --n 6144 --k 2048
    python microbench.py attention --batch 8 --context 8192
    python microbench.py attention --batch 1 --rows 2048 --context 2048
    python microbench.py norm --rows 8

Sizes default to the LFM2-8B-A1B layer (hidden 2048, 32 experts of width 1792 top-4, 32/8 heads of 64). Inputs are
larger than the 126 MB L2 or a 256 MB buffer is written between timed launches, so DRAM figures mean something; a
case holds a few GB at most and a run ends in seconds, which is what a profiler capture needs. Each run prints one
JSON line: milliseconds (median), the bytes or flops the kernel has to move or do, and the rate.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch

DEV = "cuda:0"


def timed(fn, iters: int, flush: bool = True) -> float:
    junk = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=DEV) if flush else None
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        if flush:
            junk.fill_(1.0)            # 256 MB written: nothing of the last launch is left in L2
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def runtime(prompt_product: str | None = None):
    from tandemllm_b200.parts import Runtime
    from tandemllm_b200.kernels import tensorcore
    rt = Runtime(torch.device(DEV), torch.bfloat16)
    tensorcore.enable(rt)
    if prompt_product:
        tensorcore.PROMPT_PRODUCT = prompt_product
    return rt


def expert_gemm(a) -> dict:
    """The routed experts of one layer: plan + gate/up with SwiGLU + down, for `tokens` rows."""
    from tandemllm_b200.config import PartSpec
    from tandemllm_b200.parts import make_part
    rt = runtime(a.product)
    E, H, I, k, R = a.experts, a.hidden, a.inter, a.top_k, a.tokens
    spec = PartSpec("sigmoid_topk_experts", {"num_experts": E, "top_k": k, "intermediate_size": I, "expert_bias": False,
                                             "normalize": True, "scale": 1.0,
                                             "names": {"router": "gate", "bias": "b", "experts": "experts", "gate": "w1",
                                                       "up": "w3", "down": "w2"}})
    part = make_part("feed_forward", spec, prefix="m.", hidden_size=H)
    part.runtime = rt
    part.w_router = torch.randn(E, H, device=DEV) * 0.5
    part.expert_bias = None
    part.w_gate_up = (torch.randn(E, 2 * I, H, device=DEV) * 0.02).to(torch.bfloat16)
    part.w_down = (torch.randn(E, H, I, device=DEV) * 0.02).to(torch.bfloat16)
    x = torch.randn(R, H, device=DEV).to(torch.bfloat16)
    ids, wts = part.route(x.float())
    touched = int(torch.unique(ids).numel())
    ms = timed(lambda: rt.tensorcore.experts(part, x, ids, wts), a.iters)
    nbytes = touched * 3 * I * H * 2
    flops = 2.0 * R * k * 3 * I * H
    return {"kernel": "experts (plan, gate/up + SwiGLU, down)", "tokens": R, "experts_touched": touched, "ms": ms,
            "bytes": nbytes, "GBps": nbytes / ms / 1e6, "TFLOPs": flops / ms / 1e9}


def dense_gemm(a) -> dict:
    rt = runtime(a.product)
    x = torch.randn(a.rows, a.k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device=DEV) * 0.02).to(torch.bfloat16)
    out = torch.empty(a.rows, a.n, dtype=torch.bfloat16 if a.out == "bf16" else torch.float32, device=DEV)
    ms = timed(lambda: rt.tensorcore.linear(x, w, None, out), a.iters)
    nbytes = (a.n * a.k + a.rows * a.k) * 2 + out.numel() * out.element_size()
    flops = 2.0 * a.rows * a.n * a.k
    return {"kernel": "dense product", "rows": a.rows, "n": a.n, "k": a.k, "ms": ms, "bytes": nbytes,
            "GBps": nbytes / ms / 1e6, "TFLOPs": flops / ms / 1e9}


def attention(a) -> dict:
    """`rows` query rows per request at the end of a context of `context` positions, `batch` requests."""
    from tandemllm_b200.kernels import ops
    rt = runtime()
    Hq, Hk, D, page = a.heads, a.kv_heads, a.head_dim, 16
    B, n, L = a.batch, a.rows, a.context
    pages_per = -(-L // page)
    kc = (torch.randn(B * pages_per, Hk, page, D, device=DEV) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(B * pages_per, Hk, page, D, device=DEV) * 0.5).to(torch.bfloat16)
    table = torch.arange(B * pages_per, dtype=torch.int32, device=DEV).view(B, pages_per)
    R = B * n
    q = torch.randn(R, Hq, D, device=DEV).to(torch.bfloat16)
    positions = torch.cat([torch.arange(L - n, L, dtype=torch.int32) for _ in range(B)]).to(DEV)
    starts = [b * n for b in range(B + 1)]
    step = types.SimpleNamespace(n_requests=B, max_rows_per_request=n, max_context=L, positions=positions,
                                 req_of_row=torch.arange(B, dtype=torch.int32, device=DEV).repeat_interleave(n),
                                 host={"row_start": starts})
    cache = types.SimpleNamespace(k=kc, v=vc, page_size=page)
    out = torch.empty(R, Hq, D, dtype=torch.bfloat16, device=DEV)
    if a.kernel in ("mma", "tc"):
        from tandemllm_b200.kernels import tensorcore
        tensorcore.PROMPT_ATTENTION = "tcgen05" if a.kernel == "tc" else "mma"
        tensorcore.lib().tl_attention_mma_use_tma(int(a.copies == "tma"))
        tensorcore.lib().tl_attention_tc_p_in_tensor_memory(int(a.p == "tmem"))
        fn = lambda: rt.tensorcore.attention(q, cache, table, step, D ** -0.5, None, out, rt)
    else:
        spans = ops.attention_spans(L)
        scratch = torch.empty(ops.attention_scratch_floats(R, Hq, D, spans), device=DEV)
        fn = lambda: ops.paged_attention_split(q, kc, vc, table, page, step.req_of_row, positions, D ** -0.5, None, out,
                                               scratch, spans, rt.status)
    ms = timed(fn, a.iters, flush=kc.numel() * 4 < 512 * 1024 * 1024)
    nbytes = B * L * Hk * D * 2 * 2
    flops = 4.0 * B * Hq * D * (n * (L - n) + n * (n + 1) / 2)
    return {"kernel": f"paged attention ({a.kernel})", "batch": B, "rows": n, "context": L, "ms": ms, "bytes": nbytes,
            "GBps": nbytes / ms / 1e6, "TFLOPs": flops / ms / 1e9}


def norm(a) -> dict:
    from tandemllm_b200.kernels import ops
    ops.core()
    R, H = a.rows, a.hidden
    res = torch.randn(R, H, device=DEV)
    delta = torch.randn(R, H, device=DEV)
    w = torch.ones(H, device=DEV)
    out = torch.empty(R, H, dtype=torch.bfloat16, device=DEV)
    ms = timed(lambda: ops.add_rmsnorm(res, delta, w, 1e-5, out), a.iters)
    nbytes = R * H * (4 + 4 + 4 + 2)
    return {"kernel": "residual add + RMS norm", "rows": R, "hidden": H, "ms": ms, "bytes": nbytes, "GBps": nbytes / ms / 1e6}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    e = sub.add_parser("expert_gemm")
    e.add_argument("--tokens", type=int, default=8)
    e.add_argument("--experts", type=int, default=32)
    e.add_argument("--hidden", type=int, default=2048)
    e.add_argument("--inter", type=int, default=1792)
    e.add_argument("--top-k", type=int, default=4)
    d = sub.add_parser("dense_gemm")
    d.add_argument("--rows", type=int, default=8)
    d.add_argument("--n", type=int, default=6144)
    d.add_argument("--k", type=int, default=2048)
    d.add_argument("--out", default="bf16", choices=("bf16", "fp32"))
    t = sub.add_parser("attention")
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--rows", type=int, default=1)
    t.add_argument("--context", type=int, default=8192)
    t.add_argument("--heads", type=int, default=32)
    t.add_argument("--kv-heads", type=int, default=8)
    t.add_argument("--head-dim", type=int, default=64)
    t.add_argument("--kernel", default="tc", choices=("tc", "mma", "split"),
                   help="tc: the tcgen05 kernel for prompt portions of head size 64 (decode rows go to the mma.sync kernel "
                        "either way); mma: the mma.sync kernel for everything; split: the CUDA-core kernel")
    t.add_argument("--p", default="tmem", choices=("tmem", "smem"),
                   help="the tcgen05 kernel: P as the MMA's operand from tensor memory, or through shared memory")
    t.add_argument("--copies", default="tma", choices=("tma", "cp.async"),
                   help="decoding with the mma kernel: a producer warp's TMA copies, or cp.async from every thread")
    n = sub.add_parser("norm")
    n.add_argument("--rows", type=int, default=8)
    n.add_argument("--hidden", type=int, default=2048)
    for p in (e, d):
        p.add_argument("--product", default="pair", choices=("pair", "single"),
                       help="prompt-sized products: the kernel on pairs of SMs (cta_group::2), or the one-CTA persistent kernel")
    for p in (e, d, t, n):
        p.add_argument("--iters", type=int, default=20)
    a = ap.parse_args(argv)
    result = {"expert_gemm": expert_gemm, "dense_gemm": dense_gemm, "attention": attention, "norm": norm}[a.what](a)
    print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in result.items()}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
