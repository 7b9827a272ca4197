"""Python entry points of the CUDA kernels: tensors in, launches on torch's current stream.

Each function checks what the kernel cannot (device, dtype, contiguity), passes raw pointers and the
stream handle through ctypes, and raises `KernelError` with the library's own message when a launcher
refuses its arguments. There is no fallback: a missing library is an error at load time.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load

FP32, BF16 = 0, 1
TL_BAD_ARGUMENT = 100001
# the gate activations of gated products (TL_ACT_* of csrc/common.cuh) and the router's scoring functions (TL_SCORE_*
# of csrc/route.cuh), by the names a part's spec gives them
ACTIVATIONS = {"silu": 1, "gelu": 2, "relu2": 3, "identity": 4}
SCORINGS = {"sigmoid": 0, "softmax": 1}


def activation_code(name: str) -> int:
    if name not in ACTIVATIONS:
        raise KernelError(f"gate activation {name!r}: one of {', '.join(ACTIVATIONS)}")
    return ACTIVATIONS[name]


def route_flags(normalize: bool, scoring: str = "sigmoid") -> int:
    """The routers' `normalize` argument: bit 0 = divide the chosen weights by their sum, bits 1.. = the scoring function."""
    if scoring not in SCORINGS:
        raise KernelError(f"router scoring function {scoring!r}: one of {', '.join(SCORINGS)}")
    return int(bool(normalize)) | (SCORINGS[scoring] << 1)


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return FP32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dtype} is not implemented; float32 and bfloat16 are")


_SIGNATURES = {
    "tl_embed_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "tl_add_rmsnorm": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                       c_void_p,
                       c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                       c_float, c_float, c_void_p, c_void_p, c_void_p],
    "tl_gated_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "tl_gemm_simt": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int,
                     c_int, c_int, c_void_p],
    "tl_gemm_simt_grouped": [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_void_p,
                             c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                             c_int, c_int, c_void_p],
    "tl_gemm_simt_tile_rows": [],
    "tl_short_conv": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                      c_int, c_int, c_int, c_void_p],
    "tl_short_conv_decode": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "tl_short_conv_state": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "tl_qk_prepare": [c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                      c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                      c_void_p, c_void_p],
    "tl_kv_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                    c_int, c_int, c_void_p, c_void_p],
    "tl_paged_attention_simt": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_int,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "tl_attention_spans": [c_int],
    "tl_paged_attention_split": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_int,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "tl_attention_join": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "tl_router_topk": [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p,
                       c_void_p],
    "tl_moe_max_tiles": [c_int, c_int, c_int],
    "tl_moe_plan_copies_rows": [c_int, c_int],
    "tl_moe_plan": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                    c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p],
    "tl_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "tl_argmax": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p],
    "tl_graph_capture_begin": [c_void_p],
    "tl_graph_capture_end": [c_void_p, c_void_p, c_void_p],
    "tl_graph_launch": [c_void_p, c_void_p],
    "tl_graph_destroy": [c_void_p],
    "tl_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_void_p],
    "tl_penalize": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p,
                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "tl_count_tokens": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p],
}

_core = None


def core():
    """The loaded core library with its signatures declared (built at the first call)."""
    global _core
    if _core is None:
        lib = load("core")
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = c_int
        lib.tl_last_error.restype = ctypes.c_char_p
        lib.tl_cuda_error_string.restype = ctypes.c_char_p
        lib.tl_cuda_error_string.argtypes = [c_int]
        _core = lib
    return _core


launches = 0        # kernels of this package launched so far (a launcher that starts two kernels counts both)


def check(code: int, what: str, lib=None, kernels: int = 1) -> None:
    global launches
    if code == 0:
        launches += kernels
        return
    lib = lib or core()
    if code == TL_BAD_ARGUMENT:
        raise KernelError(lib.tl_last_error().decode())
    raise KernelError(f"{what}: CUDA error {code}: {core().tl_cuda_error_string(code).decode()}")


# The current stream's handle is asked for once a launch: through torch's own C entry points where it has them (a
# fraction of a microsecond), else through `torch.cuda.current_stream()`, whose Python checks cost more than the launch.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def stream() -> int:
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on CUDA tensors only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} is {t.dtype}, expected {dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")


# ------------------------------------------------------------------------------------------ rows
def embed_rows(table: torch.Tensor, tokens: torch.Tensor, residual: torch.Tensor, status: torch.Tensor) -> None:
    _need(table, None, "embedding table"); _need(tokens, torch.int32, "tokens"); _need(residual, torch.float32, "residual")
    rows, hidden = residual.shape
    check(core().tl_embed_rows(ptr(table), ptr(tokens), ptr(residual), rows, hidden, table.shape[0],
                               dtype_code(table.dtype), ptr(status), stream()), "embed_rows")


class PartialSums:
    """A product's output still in `parts` partial sums [parts, rows, hidden] (32-bit), to be added in order and, when
    `dtype` is given, rounded to it (what the product's own reduction would have stored)."""

    def __init__(self, data: torch.Tensor, parts: int, rows: int, hidden: int, dtype: torch.dtype | None = None):
        self.data, self.parts, self.rows, self.hidden, self.dtype = data, parts, rows, hidden, dtype

    def materialize(self) -> torch.Tensor:
        parts = self.data[:self.parts * self.rows * self.hidden].view(self.parts, self.rows, self.hidden)
        total = torch.zeros_like(parts[0])
        for part in parts:
            total += part
        return total if self.dtype is None else total.to(self.dtype)


class ExpertRows:
    """A routed expert layer's output still as one row per (row, slot) pair in expert-sorted order [pairs, hidden]
    (32-bit), with what is needed to weigh and add them per row."""

    def __init__(self, rows: torch.Tensor, pos_of_pair: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, parts: int = 1):
        """`parts` > 1: `rows` is [parts, pairs, hidden], partial sums of a down projection split along k."""
        self.rows, self.pos_of_pair, self.ids, self.wts, self.parts = rows, pos_of_pair, ids, wts, parts

    def materialize(self) -> torch.Tensor:
        rows = self.rows
        if self.parts > 1:
            rows = rows[0].clone()
            for part in self.rows[1:]:
                rows += part
        out = torch.empty(self.ids.shape[0], rows.shape[-1], dtype=torch.float32, device=rows.device)
        check(core().tl_moe_combine(ptr(rows), ptr(self.pos_of_pair), ptr(self.ids), ptr(self.wts), ptr(out),
                                    out.shape[0], out.shape[1], self.ids.shape[1], stream()), "moe_combine")
        return out


def materialize(branch):
    """A branch output as a plain tensor, whatever form a part returned it in."""
    return branch.materialize() if isinstance(branch, (PartialSums, ExpertRows)) else branch


def add_rmsnorm(residual: torch.Tensor, delta, weight: torch.Tensor, eps: float, out: torch.Tensor,
                gather: torch.Tensor | None = None, out32: torch.Tensor | None = None, route: dict | None = None
                ) -> torch.Tensor:
    """residual += delta (32-bit); out = weight * rms_normalised(residual). `delta` is None, a float32 tensor, a
    `PartialSums` or an `ExpertRows`. With `gather` (int32 row indices) the output row i is computed from row
    gather[i] and the residual is left unchanged. `out32` also receives the normalised rows unrounded. `route`
    (router weights float32 [E, hidden], bias, k, normalize, scoring, floor, scale, ids, wts) also runs the router on the
    unrounded rows and fills ids int32 [rows, k] and wts float32 [rows, k]."""
    _need(residual, torch.float32, "residual"); _need(weight, torch.float32, "norm weight"); _need(out, None, "normed")
    if out32 is not None:
        _need(out32, torch.float32, "normed32")
    dense = parts = stride = 0
    rows_ptr = pos = ids = wts = None
    top_k, eparts, estride = 0, 1, 0
    if isinstance(delta, PartialSums):
        dense, parts, stride = delta.data.data_ptr(), delta.parts, delta.rows * delta.hidden
    elif isinstance(delta, ExpertRows):
        rows_ptr, pos, ids, wts, top_k = delta.rows, delta.pos_of_pair, delta.ids, delta.wts, delta.ids.shape[1]
        if delta.parts > 1:
            eparts, estride = delta.parts, delta.rows.shape[1] * delta.rows.shape[2]
    elif delta is not None:
        _need(delta, torch.float32, "delta")
        dense, parts = delta.data_ptr(), 1
    hidden = residual.shape[-1]
    n_out = out.shape[0]
    r = route or {}
    if route:
        _need(r["weight"], torch.float32, "router weight"); _need(r["ids"], torch.int32, "ids"); _need(r["wts"], torch.float32, "wts")
    check(core().tl_add_rmsnorm(
        ptr(residual), dense or None, parts, stride, ptr(rows_ptr), eparts, estride, ptr(pos), ptr(ids), ptr(wts), top_k,
        ptr(weight),
        ptr(out), ptr(out32), ptr(gather), n_out, hidden, float(eps), dtype_code(out.dtype), ptr(r.get("weight")),
        ptr(r.get("bias")), r["weight"].shape[0] if route else 0, int(r.get("k", 0)),
        route_flags(r.get("normalize", 0), r.get("scoring", "sigmoid")),
        float(r.get("floor", 0.0)), float(r.get("scale", 1.0)), ptr(r.get("ids")), ptr(r.get("wts")), stream()),
        "add_rmsnorm")
    return out


def gated_mul(gate_up: torch.Tensor, out: torch.Tensor, act: int = 1) -> torch.Tensor:
    """out = act(gate_up[:, :inter]) * gate_up[:, inter:], `act` a code of ACTIVATIONS (1: SiLU)."""
    _need(gate_up, out.dtype, "gate_up"); _need(out, None, "out")
    rows, inter = out.shape
    check(core().tl_gated_mul(ptr(gate_up), ptr(out), rows, inter, int(act), dtype_code(out.dtype), stream()), "gated_mul")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    return gated_mul(gate_up, out, ACTIVATIONS["silu"])


# ------------------------------------------------------------------------------------------ products
def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (+ bias) on the CUDA cores with 32-bit accumulation."""
    _need(x, w.dtype, "x"); _need(w, None, "w"); _need(out, None, "out")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    check(core().tl_gemm_simt(ptr(x), x.stride(0), ptr(w), w.stride(0), ptr(bias), ptr(out), out.stride(0), M, N, K,
                              dtype_code(x.dtype), dtype_code(out.dtype), stream()), "gemm_simt")
    return out


def gemm_simt_grouped(a: torch.Tensor, a_gather: torch.Tensor | None, a_div: int, w: torch.Tensor, out: torch.Tensor,
                      plan: "MoePlan", swiglu: bool | int) -> torch.Tensor:
    """Per sorted row i of the plan: out[i] = A[row(i)] @ w[expert(i)]^T, with w [E, N(*2 when swiglu), K]. `swiglu`:
    False for a plain product, True or a code of ACTIVATIONS for act(gate rows) * (up rows)."""
    _need(a, w.dtype, "a"); _need(w, None, "w"); _need(out, None, "out")
    E, n_rows_w, K = w.shape
    N = n_rows_w // 2 if swiglu else n_rows_w
    check(core().tl_gemm_simt_grouped(ptr(a), a.stride(0), ptr(a_gather), a_div, ptr(w), w.stride(1), w.stride(0),
                                      ptr(out), out.stride(0), plan.pairs, N, K, ptr(plan.tile_group),
                                      ptr(plan.tile_row0), ptr(plan.tile_rows), ptr(plan.n_tiles), plan.max_tiles,
                                      int(swiglu), dtype_code(a.dtype), dtype_code(out.dtype), stream()),
          "gemm_simt_grouped")
    return out


def simt_tile_rows() -> int:
    return core().tl_gemm_simt_tile_rows()


# ------------------------------------------------------------------------------------------ short conv
def short_conv(bcx, taps, bias, state, state_slot, req_of_row, row_start, positions, out) -> torch.Tensor:
    _need(bcx, out.dtype, "bcx"); _need(taps, torch.float32, "taps"); _need(state, torch.float32, "conv state")
    rows, hidden = out.shape
    K = taps.shape[1]
    check(core().tl_short_conv(ptr(bcx), ptr(taps), ptr(bias), ptr(state), ptr(state_slot), ptr(req_of_row),
                               ptr(row_start), ptr(positions), ptr(out), rows, hidden, K, dtype_code(out.dtype),
                               stream()), "short_conv")
    return out


def short_conv_decode(bcx, taps, bias, state, state_slot, req_of_row, positions, out, write_state: bool = True):
    """The convolution and the state's shift for a step of one row a request; `bcx` a tensor or `PartialSums`."""
    _need(taps, torch.float32, "taps"); _need(state, torch.float32, "conv state")
    rows, hidden = out.shape
    partial, parts, stride, data = None, 0, 0, None
    if isinstance(bcx, PartialSums):
        if bcx.dtype not in (None, out.dtype) or bcx.hidden != 3 * hidden or bcx.rows != rows:
            raise KernelError("short_conv_decode: partial sums of another shape or precision")
        partial, parts, stride = bcx.data, bcx.parts, bcx.rows * bcx.hidden
    else:
        _need(bcx, out.dtype, "bcx")
        data = bcx
    check(core().tl_short_conv_decode(ptr(data), ptr(partial), parts, stride, ptr(taps), ptr(bias), ptr(state),
                                      ptr(state_slot), ptr(req_of_row), ptr(positions), ptr(out), rows, hidden,
                                      taps.shape[1], dtype_code(out.dtype), int(write_state), stream()),
          "short_conv_decode")
    return out


def short_conv_state(bcx, state, state_slot, row_start, positions, requests: int, hidden: int, taps: int) -> None:
    _need(bcx, None, "bcx"); _need(state, torch.float32, "conv state")
    check(core().tl_short_conv_state(ptr(bcx), ptr(state), ptr(state_slot), ptr(row_start), ptr(positions), requests,
                                     hidden, taps, dtype_code(bcx.dtype), stream()), "short_conv_state")


# ------------------------------------------------------------------------------------------ attention
def qk_prepare(qkv, q_weight, k_weight, eps, inv_freq, rotary_dim, positions, req_of_row, block_table, page_size,
               q_out, k_cache, v_cache, k_out, v_out, num_heads, num_kv_heads, head_dim, status) -> None:
    _need(qkv, None, "qkv")
    rows = qkv.shape[0]
    max_pages = block_table.shape[1] if block_table is not None else 0
    check(core().tl_qk_prepare(ptr(qkv), qkv.stride(0), ptr(q_weight), ptr(k_weight), float(eps), ptr(inv_freq),
                               int(rotary_dim), ptr(positions), ptr(req_of_row), ptr(block_table), max_pages,
                               int(page_size), k_cache.shape[0] if k_cache is not None else 0, ptr(q_out), ptr(k_cache),
                               ptr(v_cache), ptr(k_out), ptr(v_out), rows,
                               num_heads, num_kv_heads, head_dim, dtype_code(qkv.dtype), ptr(status), stream()),
          "qk_prepare")


def kv_store(k, v, positions, req_of_row, block_table, page_size, k_cache, v_cache, status) -> None:
    _need(k, k_cache.dtype, "k"); _need(v, v_cache.dtype, "v")
    rows, Hk, D = k.shape
    check(core().tl_kv_store(ptr(k), ptr(v), ptr(positions), ptr(req_of_row), ptr(block_table), block_table.shape[1],
                             int(page_size), k_cache.shape[0], ptr(k_cache), ptr(v_cache), rows, Hk, D, dtype_code(k.dtype),
                             ptr(status), stream()), "kv_store")


def paged_attention_simt(q, k_cache, v_cache, block_table, page_size, req_of_row, positions, scale, window, out,
                         status) -> torch.Tensor:
    _need(q, k_cache.dtype, "q"); _need(out, q.dtype, "out")
    rows, Hq, D = q.shape
    Hk = k_cache.shape[1]
    check(core().tl_paged_attention_simt(ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_table), block_table.shape[1],
                                         int(page_size), k_cache.shape[0], ptr(req_of_row), ptr(positions), float(scale),
                                         int(window or 0), ptr(out), rows, Hq, Hk, D, dtype_code(q.dtype), ptr(status),
                                         stream()), "paged_attention")
    return out


def attention_spans(max_context: int) -> int:
    """Key spans the split kernel cuts a context of `max_context` positions into."""
    return core().tl_attention_spans(int(max_context))


def attention_scratch_floats(rows: int, num_heads: int, head_dim: int, n_spans: int) -> int:
    return rows * num_heads * n_spans * (head_dim + 2)


def paged_attention_split(q, k_cache, v_cache, block_table, page_size, req_of_row, positions, scale, window, out,
                          scratch, n_spans: int, status) -> torch.Tensor:
    """Attention of every row over its request's cached keys, split along the keys; `scratch` is float32 with at
    least attention_scratch_floats(rows, Hq, D, n_spans) elements and n_spans covers the longest context."""
    _need(q, k_cache.dtype, "q"); _need(out, q.dtype, "out"); _need(scratch, torch.float32, "scratch")
    rows, Hq, D = q.shape
    Hk = k_cache.shape[1]
    if scratch.numel() < attention_scratch_floats(rows, Hq, D, n_spans):
        raise KernelError(f"attention scratch of {scratch.numel()} floats, "
                          f"{attention_scratch_floats(rows, Hq, D, n_spans)} needed")
    check(core().tl_paged_attention_split(ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_table), block_table.shape[1],
                                          int(page_size), k_cache.shape[0], ptr(req_of_row), ptr(positions), float(scale),
                                          int(window or 0), ptr(out), ptr(scratch), rows, Hq, Hk, D, int(n_spans),
                                          dtype_code(q.dtype), ptr(status), stream()), "paged_attention_split",
          kernels=2 if n_spans > 1 else 1)
    return out


SPAN_KEYS = 256     # key positions per span of `paged_attention_split`


def attention_join(scratch, positions, window, out, n_spans: int, span_keys: int = SPAN_KEYS) -> None:
    """Adds the key spans (of `span_keys` positions each) another kernel left in `scratch` (layout of
    `paged_attention_split`) into `out`."""
    rows, Hq, D = out.shape
    check(core().tl_attention_join(ptr(scratch), ptr(positions), int(window or 0), ptr(out), rows, Hq, D, int(n_spans),
                                   int(span_keys), dtype_code(out.dtype), stream()), "attention_join",
          kernels=1 if n_spans > 1 else 0)


# ------------------------------------------------------------------------------------------ experts
def router_topk(logits, bias, k: int, normalize: bool, floor: float, scale: float, ids, wts, scoring: str = "sigmoid") -> None:
    _need(logits, torch.float32, "router logits"); _need(ids, torch.int32, "ids"); _need(wts, torch.float32, "weights")
    rows, E = logits.shape
    check(core().tl_router_topk(ptr(logits), logits.stride(0), ptr(bias), rows, E, k, route_flags(normalize, scoring), float(floor),
                                float(scale), ptr(ids), ptr(wts), stream()), "router_topk")


class MoePlan:
    """Device buffers of one routing plan: pairs sorted by expert and the map of row tiles."""

    def __init__(self, max_pairs: int, num_experts: int, tile_rows: int, device):
        self.num_experts, self.tile_m, self.max_pairs = num_experts, tile_rows, max_pairs
        self.max_tiles_cap = core().tl_moe_max_tiles(max_pairs, num_experts, tile_rows)
        i32 = dict(dtype=torch.int32, device=device)
        self.counts = torch.zeros(num_experts, **i32)
        self.offsets = torch.zeros(num_experts + 1, **i32)
        self.sorted_pairs = torch.zeros(max(max_pairs, 1), **i32)
        self.pos_of_pair = torch.zeros(max(max_pairs, 1), **i32)
        self.tile_group = torch.zeros(self.max_tiles_cap, **i32)
        self.tile_row0 = torch.zeros(self.max_tiles_cap, **i32)
        self.tile_rows = torch.zeros(self.max_tiles_cap, **i32)
        self.n_tiles = torch.zeros(1, **i32)
        self.block_hist = torch.zeros(-(-max(max_pairs, 1) // 256) * num_experts, **i32)    # per-chunk counts
        self.pairs = 0
        self.max_tiles = 1

    def build(self, ids: torch.Tensor, x: torch.Tensor | None = None, x_sorted: torch.Tensor | None = None) -> "MoePlan":
        """Build the plan for `ids` [rows, k]. With `x` [rows, width] (bfloat16) and `x_sorted` [pairs, width], the
        token rows are copied into expert-sorted order as well when the one-kernel form applies; `self.copied`
        says whether they were."""
        pairs = ids.numel()
        if pairs > self.max_pairs:
            raise KernelError(f"routing plan sized for {self.max_pairs} pairs, got {pairs}")
        self.pairs = pairs
        self.max_tiles = core().tl_moe_max_tiles(pairs, self.num_experts, self.tile_m)
        launched = ctypes.c_int(0)
        check(core().tl_moe_plan(ptr(ids), pairs, self.num_experts, self.tile_m, ids.shape[-1], ptr(self.counts),
                                 ptr(self.offsets), ptr(self.sorted_pairs), ptr(self.pos_of_pair), ptr(self.tile_group),
                                 ptr(self.tile_row0), ptr(self.tile_rows), ptr(self.n_tiles), ptr(self.block_hist), ptr(x),
                                 x.stride(0) if x is not None else 0, ptr(x_sorted), x.shape[1] if x is not None else 0,
                                 ctypes.addressof(launched), stream()), "moe_plan", kernels=0)
        global launches
        launches += launched.value
        self.copied = x is not None and bool(core().tl_moe_plan_copies_rows(pairs, self.num_experts))
        return self


def moe_combine(y, plan: MoePlan, ids, wts, out) -> torch.Tensor:
    _need(y, torch.float32, "expert outputs"); _need(out, torch.float32, "out")
    rows, hidden = out.shape
    check(core().tl_moe_combine(ptr(y), ptr(plan.pos_of_pair), ptr(ids), ptr(wts), ptr(out), rows, hidden, ids.shape[1],
                                stream()), "moe_combine")
    return out


# ------------------------------------------------------------------------------------------ CUDA graphs
class DeviceGraph:
    """A captured CUDA graph on the runtime API (csrc/graphs.cu says why not `torch.cuda.CUDAGraph`). Between
    `capture_begin` and `capture_end` the current stream captures and this thread's allocations come from `pool` (a
    `torch.cuda.MemPool` that the caller keeps as long as any graph captured into it may be replayed): what a captured
    kernel writes stays where it is until the tensor that holds it is dropped, and the memory of tensors dropped since is
    used again by later captures into the same pool, whose graphs therefore must not be replayed side by side."""

    def __init__(self):
        self._exec = ctypes.c_void_p(None)
        self._pool_context = None
        self._stream = None
        self.nodes = 0

    def capture_begin(self, pool) -> None:
        self._stream = stream()
        self._pool_context = torch.cuda.use_mem_pool(pool)
        self._pool_context.__enter__()
        try:
            check(core().tl_graph_capture_begin(self._stream), "graph capture", kernels=0)
        except BaseException:
            self._pool_context.__exit__(None, None, None)
            self._pool_context = None
            raise

    def capture_end(self) -> None:
        nodes = ctypes.c_int(0)
        try:
            code = core().tl_graph_capture_end(self._stream, ctypes.byref(self._exec), ctypes.byref(nodes))
        finally:
            self._pool_context.__exit__(None, None, None)
            self._pool_context = None
        check(code, "graph capture", kernels=0)
        self.nodes = nodes.value

    def replay(self) -> None:
        check(core().tl_graph_launch(self._exec, stream()), "graph launch", kernels=0)

    def __del__(self):
        ex, self._exec = self._exec, ctypes.c_void_p(None)
        if ex and _core is not None:
            _core.tl_graph_destroy(ex)


# ------------------------------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(logits, torch.float32, "logits"); _need(out, torch.int32, "out")
    rows, V = logits.shape
    check(core().tl_argmax(ptr(logits), logits.stride(0), rows, V, ptr(out), stream()), "argmax")
    return out


def sample(logits, temperature, top_k, top_p, min_p, seed, position, out) -> torch.Tensor:
    _need(logits, torch.float32, "logits"); _need(temperature, torch.float32, "temperature")
    _need(top_k, torch.int32, "top_k"); _need(top_p, torch.float32, "top_p"); _need(min_p, torch.float32, "min_p")
    _need(seed, torch.int64, "seed"); _need(position, torch.int32, "position"); _need(out, torch.int32, "out")
    rows, V = logits.shape
    check(core().tl_sample(ptr(logits), logits.stride(0), rows, V, ptr(temperature), ptr(top_k), ptr(top_p), ptr(min_p),
                           ptr(seed), ptr(position), ptr(out), stream()), "sample")
    return out


def penalize(logits, counts, slot, repetition, presence, frequency, bias=None) -> torch.Tensor:
    """Penalties and added logits, in place on float32 logits [n, V]. `counts` int32 [slots, V] (None when no row
    has penalties); `slot` int32 [n], negative for a row without penalties; `repetition`, `presence`, `frequency`
    float32 [n]; `bias` None or (begin int32 [n + 1], token int32 [m], value float32 [m])."""
    _need(logits, torch.float32, "logits"); _need(slot, torch.int32, "slot")
    _need(repetition, torch.float32, "repetition"); _need(presence, torch.float32, "presence")
    _need(frequency, torch.float32, "frequency")
    rows, V = logits.shape
    slots, counts_ld, counts_ptr = 0, 0, None
    if counts is not None:
        _need(counts, torch.int32, "counts")
        slots, counts_ld, counts_ptr = counts.shape[0], counts.stride(0), ptr(counts)
        if counts.shape[1] != V:
            raise ValueError(f"counts over {counts.shape[1]} tokens for logits over {V}")
    begin = token = value = None
    if bias is not None:
        _need(bias[0], torch.int32, "bias begin"); _need(bias[1], torch.int32, "bias token")
        _need(bias[2], torch.float32, "bias value")
        if bias[0].numel() != rows + 1 or bias[1].numel() != bias[2].numel():
            raise ValueError("bias: begin needs one entry a row and one more, and a value for every token")
        begin, token, value = ptr(bias[0]), ptr(bias[1]), ptr(bias[2])
    check(core().tl_penalize(ptr(logits), logits.stride(0), rows, V, counts_ptr, counts_ld, slots, ptr(slot),
                             ptr(repetition), ptr(presence), ptr(frequency), begin, token, value, stream()), "penalize")
    return logits


def count_tokens(counts: torch.Tensor, tokens: torch.Tensor, slot) -> None:
    """counts[slot, token] += 1 for int32 tokens [n]; `slot` is an int32 tensor [n] or one row's index."""
    _need(counts, torch.int32, "counts"); _need(tokens, torch.int32, "tokens")
    slots, V = counts.shape
    if isinstance(slot, torch.Tensor):
        _need(slot, torch.int32, "slot")
        if slot.numel() != tokens.numel():
            raise ValueError(f"{slot.numel()} slots for {tokens.numel()} tokens")
        slot_ptr, one = ptr(slot), -1
    else:
        slot_ptr, one = None, int(slot)
    check(core().tl_count_tokens(ptr(counts), counts.stride(0), slots, V, slot_ptr, one, ptr(tokens), tokens.numel(),
                                 stream()), "count_tokens")
