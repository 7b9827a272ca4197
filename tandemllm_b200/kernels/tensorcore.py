"""The bfloat16 path's tensor-core kernels (tcgen05 + TMA, `csrc/tc_gemm.cu`): when a runtime has them,
`parts.linear` and the expert feed-forward send their products here.

Choice of kernel by shape:
  up to 32 token rows and 64 MB of weights (a decode step's projections): `csrc/gemm_skinny_mma.cu`, which loads
                         both operands straight into mma.sync registers; such a product's time is the length of its
                         chain of dependent steps, and this chain is the shortest.
  up to 128 token rows   the swapped orientation: 128 weight rows on the MMA's M side, the tokens (padded to 16,
                         32, 64 or 128) on its N side, so a decode step streams every weight once. When a product
                         would launch fewer CTAs than the GPU has SMs, its k range is split over several CTAs that
                         write 32-bit partial sums to a workspace; they are added in a fixed order by a second
                         kernel, or, for a branch's last product, by the norm kernel that consumes the branch
                         (`ops.PartialSums`).
  more rows              the persistent kernel: one CTA an SM walks over tiles of 128 token rows by 256 weight rows,
                         its loads, its MMAs and its epilogue running side by side on two accumulators.
Experts: the plan's tiles carry the expert, gate/up and SwiGLU run in one kernel, the down projection writes 32-bit
rows that the next norm kernel weighs and adds (`ops.ExpertRows`). A step of up to 16 rows runs both products in the
grouped form of the register-only kernel (plan tiles of 8 rows; with at most 16 pairs no plan at all: the CTAs find each
expert's pairs in the ids). Above that the tcgen05 kernels: with a row or two an expert the gate/up product fetches each
token row by its index; with more, the rows are copied into expert-sorted order first (by the plan kernel itself for
a small step).
A short-convolution mixer's in-projection of up to 8 decode rows runs with the convolution and the state's shift in its
epilogue (`in_proj_conv`). Attention (`csrc/attention_mma.cu`) is dispatched from here as well.
Anything the kernels do not take (k or a row stride not a multiple of 8 elements, as TMA needs 16-byte strides)
goes back to the CUDA-core kernels by returning None.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p

import torch

from ..settings import SETTINGS
from . import ops
from .build import load

SKINNY_TOKENS = 32              # up to this many token rows ...
SKINNY_K = 2048                 # ... of at most this many elements (one round of loads a warp) ...
SKINNY_BYTES = 64 << 20         # ... against at most this many bytes of weights go to the register-only kernel
SKINNY_ROWS = 16                # rows of a step up to which the experts go to its grouped form, over plan tiles of 8 (an
                                # expert with more pairs has two tiles, and the second reads its weights from L2); measured
                                # against the tcgen05 form: 8 % faster a step at 16 rows, even at 24, 4 % slower at 32
SKINNY_PAIRS = 24               # routed pairs of such a step up to which its products run without a routing plan
PROMPT_ATTENTION = "tcgen05"    # prompt portions of head size 64: the tcgen05 kernel (csrc/attention_tc.cu), or "mma" for the
                                # mma.sync kernel that also takes them (kept for head size 128 and for comparison)
# prompt-sized products on pairs of SMs (csrc/tc_gemm_pair.cu), or "single": the one-CTA persistent kernel of
# csrc/tc_gemm.cu (kept for comparison and as the pair's reference)
PROMPT_PRODUCT = SETTINGS.get("PROMPT_PRODUCT")
if PROMPT_PRODUCT not in ("pair", "single"):
    raise ValueError(f"TANDEMLLM_PROMPT_PRODUCT={PROMPT_PRODUCT!r}: pair or single")
PAIR_HALF_ROWS = 64             # rows an expert (on average) up to which the experts' pair products run two CTAs an SM
_lib = None


def lib():
    global _lib
    if _lib is None:
        l = load("tensorcore")
        l.tl_gemm_tc.argtypes = [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p,
                                 c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]
        l.tl_gemm_tc.restype = c_int
        l.tl_gemm_tc_pair.argtypes = [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p,
                                      c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
        l.tl_gemm_tc_pair.restype = c_int
        l.tl_tc_pair_token_tile.argtypes = [c_int]
        l.tl_tc_pair_token_tile.restype = c_int
        l.tl_gather_rows.argtypes = [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]
        l.tl_gather_rows.restype = c_int
        l.tl_tc_token_tile.argtypes = [c_int, c_int]
        l.tl_tc_token_tile.restype = c_int
        l.tl_tc_last_error.restype = ctypes.c_char_p
        l.tl_paged_attention_mma.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                             c_void_p, ctypes.c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                             c_int, c_void_p, c_void_p]
        l.tl_paged_attention_mma.restype = c_int
        l.tl_paged_attention_tc.argtypes = l.tl_paged_attention_mma.argtypes
        l.tl_paged_attention_tc.restype = c_int
        l.tl_attention_tc_tile_rows.argtypes = [c_int, c_int]
        l.tl_attention_tc_tile_rows.restype = c_int
        l.tl_attention_tc_supported.argtypes = [c_int, c_int, c_int, c_int]
        l.tl_attention_tc_supported.restype = c_int
        l.tl_attention_tc_p_in_tensor_memory.argtypes = [c_int]
        l.tl_attention_tc_p_in_tensor_memory.restype = None
        l.tl_attention_mma_use_tma.argtypes = [c_int]
        l.tl_attention_mma_use_tma.restype = None
        l.tl_attention_mma_tile_rows.argtypes = [c_int, c_int]
        l.tl_attention_mma_tile_rows.restype = c_int
        l.tl_attention_mma_supported.argtypes = [c_int, c_int, c_int]
        l.tl_attention_mma_supported.restype = c_int
        l.tl_gemm_skinny_supported.argtypes = [c_int, c_int, c_int, c_longlong, c_longlong]
        l.tl_gemm_skinny_supported.restype = c_int
        l.tl_gemm_skinny_mma.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int,
                                         c_int, c_int, c_int, c_void_p]
        l.tl_gemm_skinny_mma.restype = c_int
        l.tl_gemm_skinny_grouped.argtypes = [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_void_p,
                                             c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]
        l.tl_gemm_skinny_grouped.restype = c_int
        l.tl_gemm_skinny_conv.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
        l.tl_gemm_skinny_conv.restype = c_int
        _lib = l
    return _lib


def _check(code: int, what: str, kernels: int = 1) -> None:
    if code == 0:
        ops.launches += kernels
        return
    if code == ops.TL_BAD_ARGUMENT:
        raise ops.KernelError(lib().tl_tc_last_error().decode())
    raise ops.KernelError(f"{what}: CUDA error {code}: {ops.core().tl_cuda_error_string(code).decode()}")


def _pow2_at_least(n: int, lo: int = 16) -> int:
    b = lo
    while b < n:
        b *= 2
    return b


def usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    K = x.shape[-1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(-1) == 1
            and w.stride(-1) == 1 and x.stride(0) % 8 == 0 and w.stride(-2) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


class TensorCore:
    def __init__(self, device, status: torch.Tensor):
        self.device, self.status = device, status
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self._workspace = None
        self._pair_order = None
        self._pairs = None
        self._outgrown = []

    def workspace(self, floats: int) -> torch.Tensor:
        if self._workspace is None or self._workspace.numel() < floats:
            if self._workspace is not None:
                self._outgrown.append(self._workspace)      # a captured decode graph may still write to the smaller one
            self._workspace = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=self.device)
        return self._workspace

    # ---- x @ w^T (+ bias) ----
    def gemm(self, x, w2d, bias, out, *, rows_per_group=0, plan=None, swiglu=False, swap=None, bn=None, n_out=None,
             defer: bool = False, row_index=None, row_div: int = 1, rows: int | None = None, splits: int = 1):
        """Runs the product into `out`. With `defer`, a product that was split along k is left as partial sums and
        returned as `ops.PartialSums` (nothing is written to `out`); otherwise returns None. With `row_index` (grouped,
        swapped) the plan's position i stands for row row_index[i] // row_div of x, and `rows` is the number of
        positions."""
        M, K = (rows if rows is not None else x.shape[0]), x.shape[1]
        N = n_out if n_out is not None else w2d.shape[0]
        if swap is None:
            swap = M <= 128
        if bn is None:
            bn = _pow2_at_least(M) if swap else 256        # 256 without swap: the persistent kernel
        if (PROMPT_PRODUCT == "pair" and not swap and bn == 256 and splits == 1 and row_index is None
                and (plan is None or plan.tile_m <= lib().tl_tc_pair_token_tile(1))):
            if defer and plan is None and not swiglu and out.dtype == torch.float32:
                # A portion of a few hundred rows has fewer tiles than the GPU has pairs of SMs, and a pair streams its
                # tile at the rate of two SMs whatever else is idle: the reduction is cut into runs, each a work item
                # with partial sums of its own, which the norm kernel behind adds.
                tiles, kb = -(-N // 256) * -(-M // 256), -(-K // 64)
                runs = min(self.pairs() // tiles, kb // 4, 8)
                if runs > 1:
                    runs = -(-kb // -(-kb // runs))            # no run is empty
                    partial = self.workspace(runs * M * N)
                    self.gemm_pair(x, w2d, bias, partial[:runs * M * N].view(runs * M, N), n_out=n_out, rows=rows,
                                   splits=runs)
                    return ops.PartialSums(partial, runs, M, N, None)
            self.gemm_pair(x, w2d, bias, out, rows_per_group=rows_per_group, plan=plan, gated=int(swiglu), n_out=n_out,
                           rows=rows)
            return None
        forced, partial = splits > 1, None
        if forced:
            partial = out           # the caller's [splits, M, N] partial sums begin at `out`; the caller adds them
        elif swap and plan is None and not swiglu:
            ctas = -(-N // 128) * -(-M // bn)
            kb = -(-K // 64)
            if ctas < self.sm_count and kb >= 8:
                splits = max(1, min(kb // 4, -(-self.sm_count // ctas), 16))
                if splits > 1:
                    partial = self.workspace(splits * M * N)
        # `defer` True: a 32-bit result may stay in partial sums; "rounded": so may one of any precision, and its
        # consumer rounds the sum to the output's precision
        deferred = forced or (bool(defer) and splits > 1 and (out.dtype == torch.float32 or defer == "rounded"))
        tg = tr0 = trs = nt = None
        max_tiles = 0
        if plan is not None:
            tg, tr0, trs, nt, max_tiles = plan.tile_group, plan.tile_row0, plan.tile_rows, plan.n_tiles, plan.max_tiles
        code = lib().tl_gemm_tc(
            x.data_ptr(), x.stride(0), x.shape[0], w2d.data_ptr(), w2d.stride(0), w2d.shape[0], rows_per_group,
            ops.ptr(bias), out.data_ptr(), out.stride(0), M, N, K, int(swap), bn, int(swiglu), ops.dtype_code(out.dtype),
            ops.ptr(tg), ops.ptr(tr0), ops.ptr(trs), ops.ptr(nt), max_tiles, ops.ptr(row_index), int(row_div), splits,
            ops.ptr(partial), int(not deferred),
            self.status.data_ptr(), ops.stream())
        _check(code, "gemm_tc", kernels=2 if splits > 1 and not deferred else 1)
        if not deferred or forced:
            return None
        return ops.PartialSums(partial, splits, M, N, None if out.dtype == torch.float32 else out.dtype)

    def pairs(self) -> int:
        """Pairs of CTAs of the plain pair product that the GPU holds at a time, one CTA an SM."""
        if self._pairs is None:
            self._pairs = max(1, int(lib().tl_tc_pair_resident(0, 1)))
        return self._pairs

    def gemm_pair(self, x, w2d, bias, out, *, rows_per_group=0, plan=None, gated: int = 0, n_out=None,
                  rows: int | None = None, per_sm: int | None = None, splits: int = 1) -> None:
        """The product on pairs of SMs (csrc/tc_gemm_pair.cu): 256 outputs by up to 256 token rows a pair, the N side
        of its MMAs as many rows as a tile holds. `plan`: tiles of any height up to 256 rows. `per_sm` 2: two CTAs an
        SM, each with half the shared and tensor memory (gated: tiles of up to 128 rows), the form for products bound
        by their weights; default: 2 for a plan with tiles of up to 128 rows, else 1. `splits` > 1: `out` is
        [splits, M, N] 32-bit and receives the partial results of as many runs of k-blocks (plain product only)."""
        M, K = (rows if rows is not None else x.shape[0]), x.shape[1]
        N = n_out if n_out is not None else w2d.shape[0]
        tg = tr0 = trs = nt = None
        max_tiles = plan_rows = 0
        if plan is not None:
            tg, tr0, trs, nt, max_tiles, plan_rows = (plan.tile_group, plan.tile_row0, plan.tile_rows, plan.n_tiles,
                                                      plan.max_tiles, plan.tile_m)
        if per_sm is None:
            per_sm = 2 if plan is not None and plan.tile_m <= 128 else 1
        _check(lib().tl_gemm_tc_pair(x.data_ptr(), x.stride(0), x.shape[0], w2d.data_ptr(), w2d.stride(0), w2d.shape[0],
                                     rows_per_group, ops.ptr(bias), out.data_ptr(), out.stride(0), M, N, K, int(gated),
                                     ops.dtype_code(out.dtype), ops.ptr(tg), ops.ptr(tr0), ops.ptr(trs), ops.ptr(nt),
                                     max_tiles, plan_rows, per_sm, splits, self.status.data_ptr(), ops.stream()),
               "gemm_tc_pair")

    def gated(self, x, w_gate_up, out, act: int = 1) -> bool:
        """out = act(x gate^T) * (x up^T) for w_gate_up = [gate rows; up rows], in the persistent kernel with the gated
        epilogue (`act`: a code of ops.ACTIVATIONS, 1 = SiLU); False (nothing done) for a decode step's few rows or
        operands the kernels do not take."""
        inter = w_gate_up.shape[0] // 2
        if x.shape[0] <= 128 or not usable(x, w_gate_up) or inter % 8 or out.stride(-1) != 1 or out.dtype != torch.bfloat16:
            return False
        self.gemm(x, w_gate_up, None, out, swiglu=act, swap=False, n_out=inter)
        return True

    def linear(self, x, w, bias, out, defer: bool = False):
        """False when the kernels do not take these operands; else True, or the deferred partial sums."""
        if not usable(x, w) or out.stride(-1) != 1:
            return False
        M, K = x.shape
        N = w.shape[0]
        if (M <= SKINNY_TOKENS and K <= SKINNY_K and N * K * 2 <= SKINNY_BYTES
                and lib().tl_gemm_skinny_supported(M, N, K, x.stride(0), w.stride(0))):
            # a few tokens against some MB of weights: the kernel with the shortest chain of dependent steps
            _check(lib().tl_gemm_skinny_mma(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), ops.ptr(bias),
                                            out.data_ptr(), out.stride(0), M, N, K, ops.dtype_code(out.dtype),
                                            ops.stream()), "gemm_skinny_mma")
            return True
        return self.gemm(x, w, bias, out, defer=defer) or True

    def in_proj_conv(self, x, w_in, b_in, taps, b_taps, state, state_slot, req_of_row, positions, y,
                     write_state: bool = True) -> bool:
        """A short-convolution mixer's in-projection and convolution of a decode step of at most 8 rows (one row a
        request) in one kernel: the same bits as `linear` into bfloat16 followed by `ops.short_conv_decode`. False
        when the shapes are not those of the register-only product."""
        M, K = x.shape
        H = y.shape[1]
        if (M > 8 or not usable(x, w_in) or K > SKINNY_K or 3 * H * K * 2 > SKINNY_BYTES or w_in.shape[0] != 3 * H
                or y.dtype != torch.bfloat16 or not y.is_contiguous() or taps.dtype != torch.float32
                or not taps.is_contiguous() or state.dtype != torch.float32 or not state.is_contiguous()
                or not lib().tl_gemm_skinny_supported(M, 3 * H, K, x.stride(0), w_in.stride(0))):
            return False
        _check(lib().tl_gemm_skinny_conv(x.data_ptr(), x.stride(0), w_in.data_ptr(), w_in.stride(0), ops.ptr(b_in),
                                         taps.data_ptr(), ops.ptr(b_taps), state.data_ptr(), state_slot.data_ptr(),
                                         req_of_row.data_ptr(), positions.data_ptr(), y.data_ptr(), M, H, K, taps.shape[1],
                                         int(write_state), ops.stream()), "gemm_skinny_conv")
        return True

    # ---- routed experts ----
    def expert_tile(self, pairs: int, experts: int) -> tuple[bool, int, int]:
        """(swapped?, token tile of the MMA's N side, rows of a plan tile) for `pairs` pairs over `experts` experts."""
        avg = pairs / experts
        swap = avg <= 48
        bn = 16 if avg <= 12 else 32 if avg <= 24 else 64 if swap else 256
        if not swap and PROMPT_PRODUCT == "pair":
            # few rows an expert: the products are bound by the experts' weights, and run two CTAs an SM on tiles of 128
            return swap, bn, lib().tl_tc_pair_token_tile(2 if avg <= PAIR_HALF_ROWS else 1)
        return swap, bn, lib().tl_tc_token_tile(int(swap), bn)

    def _experts_of_a_tiny_step(self, part, x, ids, wts, plan):
        """Up to SKINNY_ROWS rows: a few experts' weights and nothing else to read, so the product whose CTAs are many
        and start at once (16 outputs each, operands straight into registers, all loads in flight) beats the tcgen05
        one, whose CTAs of 128 outputs are few and each wait for a TMA ring to fill. The plan is built in tiles of 8 rows,
        which is what a CTA of that product takes."""
        E, I2, H = part.w_gate_up.shape
        inter, (R, k) = I2 // 2, ids.shape
        P = R * k
        act = torch.empty(P, inter, dtype=x.dtype, device=x.device)
        y = torch.empty(P, H, dtype=torch.float32, device=x.device)
        if plan is None and part.load is None and P <= SKINNY_PAIRS and R <= 8 and ids.is_contiguous():
            # No plan: the products' CTAs find each expert's pairs in the ids themselves, rows stay in pair order (a CTA
            # takes all of an expert's pairs, at most 8 rows: a row chooses an expert once, so up to 8 rows of a step). A
            # pair whose expert an earlier pair has costs CTAs that start, look and leave in between the working ones.
            # Measured a step of 22 expert layers, top-4 of 32 experts, against the plan: 97 us gained with 4 pairs, 82 with
            # 8, 33 with 16; 26 lost with 24, 74 with 32 while a CTA a pair looked for its group's earlier pairs. Now that
            # the CTAs with work are the grid's first (up to 32 pairs, see the kernel): 832 -> 881 tok/s at batch 1, even
            # at 16 pairs, 2854 -> 2869 tok/s at 24 pairs, 3434 -> 3388 at 32.
            where = (None, None, None, None, 0, ids.data_ptr(), P, E)
            gate_up_rows, pos, div = None, self.pair_order(), k
        else:
            if plan is None or plan.tile_m != 8:
                plan = part.plan_for(P, x.device, 8).build(ids)
            if part.load is not None:
                part.load.add_(plan.counts)
            where = (plan.tile_group.data_ptr(), plan.tile_row0.data_ptr(), plan.tile_rows.data_ptr(),
                     plan.n_tiles.data_ptr(), plan.max_tiles, None, 0, E)
            gate_up_rows, pos, div = plan.sorted_pairs.data_ptr(), plan.pos_of_pair, k
        _check(lib().tl_gemm_skinny_grouped(x.data_ptr(), x.stride(0), gate_up_rows, div,
                                            part.w_gate_up.data_ptr(), H, I2, act.data_ptr(), inter, inter, H, part.act,
                                            ops.dtype_code(act.dtype), *where, self.status.data_ptr(), ops.stream()),
               "gemm_skinny_grouped")
        _check(lib().tl_gemm_skinny_grouped(act.data_ptr(), inter, None, 1, part.w_down.data_ptr(), inter, H, y.data_ptr(), H,
                                            H, inter, 0, ops.dtype_code(y.dtype), *where, self.status.data_ptr(),
                                            ops.stream()), "gemm_skinny_grouped")
        return ops.ExpertRows(y, pos, ids, wts)

    def pair_order(self) -> torch.Tensor:
        """0, 1, 2, ...: the places of expert rows that were left in the order of their pairs."""
        if self._pair_order is None:
            self._pair_order = torch.arange(SKINNY_PAIRS, dtype=torch.int32, device=self.device)
        return self._pair_order

    def experts(self, part, x, ids, wts, plan=None):
        """The routed experts of `part` on rows x: an `ops.ExpertRows` (to be weighed and added per row), or None
        when the kernels do not take the shapes. `plan`: the routing plan when something built it already."""
        E, I2, H = part.w_gate_up.shape
        inter = I2 // 2
        if not usable(x, part.w_gate_up.view(E * I2, H)) or inter % 8 or not part.w_down.is_contiguous():
            return None
        R, k = ids.shape
        P = R * k
        if R <= SKINNY_ROWS and H % 8 == 0:
            return self._experts_of_a_tiny_step(part, x, ids, wts, plan)
        swap, bn, tile = self.expert_tile(P, E)
        fetch = swap and P <= 2 * E           # a row or two a tile: the gate/up product fetches each token row by its index
        xs = None
        if plan is None or plan.tile_m != tile:
            plan = part.plan_for(P, x.device, tile)
            if fetch:
                plan.build(ids)
            else:
                xs = torch.empty(P, H, dtype=x.dtype, device=x.device)
                if not plan.build(ids, x, xs).copied:      # the one-kernel plan of a small step copies the rows as well
                    _check(lib().tl_gather_rows(x.data_ptr(), x.stride(0), plan.sorted_pairs.data_ptr(), k, xs.data_ptr(),
                                                P, H, ops.stream()), "gather_rows")
        elif not fetch:
            xs = torch.empty(P, H, dtype=x.dtype, device=x.device)
            _check(lib().tl_gather_rows(x.data_ptr(), x.stride(0), plan.sorted_pairs.data_ptr(), k, xs.data_ptr(), P, H,
                                        ops.stream()), "gather_rows")
        if part.load is not None:
            part.load.add_(plan.counts)
        act = torch.empty(P, inter, dtype=x.dtype, device=x.device)
        w_gate_up = part.w_gate_up.view(E * I2, H)
        if fetch:
            self.gemm(x, w_gate_up, None, act, rows_per_group=I2, plan=plan, swiglu=part.act, swap=True, bn=bn, n_out=inter,
                      row_index=plan.sorted_pairs, row_div=k, rows=P)
        else:
            self.gemm(xs, w_gate_up, None, act, rows_per_group=I2, plan=plan, swiglu=part.act, swap=swap, bn=bn, n_out=inter)
        w_down = part.w_down.view(E * H, inter)
        ctas = min(P, E) * -(-H // 128)
        if fetch and ctas < self.sm_count and inter >= 512:
            # as few pairs: the down product is split along k as well, and the norm kernel adds its partial sums
            splits = max(2, min(-(-inter // 64) // 4, -(-self.sm_count // ctas), 16))
            y = self.workspace(splits * P * H)[:splits * P * H].view(splits, P, H)
            self.gemm(act, w_down, None, y[0], rows_per_group=H, plan=plan, swap=True, bn=bn, n_out=H, splits=splits)
            return ops.ExpertRows(y, plan.pos_of_pair, ids, wts, parts=splits)
        y = torch.empty(P, H, dtype=torch.float32, device=x.device)
        self.gemm(act, w_down, None, y, rows_per_group=H, plan=plan, swap=swap, bn=bn, n_out=H)
        return ops.ExpertRows(y, plan.pos_of_pair, ids, wts)


    # ---- attention ----
    def query_tiles(self, step, tile_rows: int) -> torch.Tensor:
        """int32 [tiles, 3] = (request, first row, rows) cutting every request's rows of this step into tiles of at
        most `tile_rows` query rows. A decode-only step (one row a request) is laid out by device code alone, so
        that it can be captured in a graph; anything else comes from the step's host lists. Kept on the step."""
        key = ("query_tiles", tile_rows)
        if key not in step.host:
            B = step.n_requests
            if step.max_rows_per_request == 1:
                ar = torch.arange(B, dtype=torch.int32, device=self.device)
                step.host[key] = torch.stack([ar, ar, torch.ones_like(ar)], 1).contiguous()
            else:
                starts = step.host["row_start"]
                rows = [(b, r0, min(tile_rows, starts[b + 1] - r0)) for b in range(B)
                        for r0 in range(starts[b], starts[b + 1], tile_rows)]
                step.host[key] = torch.tensor(rows, dtype=torch.int32).to(self.device, non_blocking=True)
        return step.host[key]

    def attention(self, q, cache, table, step, scale, window, out, runtime) -> bool:
        """Attention of every row over its request's cached keys on the tensor cores; False when the sizes are not
        the kernel's (head sizes 64 and 128, groups up to 64): the caller then uses the CUDA-core kernel."""
        R, Hq, D = q.shape
        Hk = cache.k.shape[1]
        if q.dtype != torch.bfloat16 or not lib().tl_attention_mma_supported(Hq, Hk, D):
            return False
        G = Hq // Hk
        if (PROMPT_ATTENTION == "tcgen05" and step.max_rows_per_request * G > 16
                and lib().tl_attention_tc_supported(Hq, Hk, D, cache.page_size)):
            return self._prompt_attention(q, cache, table, step, scale, window, out, runtime)
        tile_rows = lib().tl_attention_mma_tile_rows(Hq, Hk)
        tiles = self.query_tiles(step, tile_rows)
        n_tiles = tiles.shape[0]
        # Few tiles and long contexts (decoding): split the keys over CTAs as well, in spans long enough that a CTA's
        # start-up is a small part of its work and short enough that the grid still has a few CTAs per SM.
        span_keys = 0
        ctas, slots = n_tiles * Hk, 3 * self.sm_count         # about three CTAs of the decode form run on an SM at once
        if step.max_context > 512 and 2 * ctas <= slots:
            # a handful of requests: as many spans as fill the GPU once, so that nobody runs in a second, thin wave
            span_keys = max(256, -(-(-(-step.max_context // (slots // ctas))) // 64) * 64)
        elif step.max_context > 512 and ctas < 8 * self.sm_count:
            span_keys = 256
            while span_keys < 2048 and ctas * -(-step.max_context // (2 * span_keys)) >= 4 * self.sm_count:
                span_keys *= 2
        spans = -(-step.max_context // span_keys) if span_keys else 1
        if spans <= 1:
            span_keys, spans = 0, 1
        scratch = runtime.scratch("attention", ops.attention_scratch_floats(R, Hq, D, spans)) if span_keys else None
        code = lib().tl_paged_attention_mma(
            q.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(), table.data_ptr(), table.shape[1], cache.page_size,
            cache.k.shape[0], tiles.data_ptr(), n_tiles, min(tile_rows, step.max_rows_per_request), step.positions.data_ptr(),
            float(scale), int(window or 0), out.data_ptr(), ops.ptr(scratch), R, Hq, Hk, D, spans, span_keys, self.status.data_ptr(), ops.stream())
        _check(code, "attention_mma")
        if span_keys:
            ops.attention_join(scratch, step.positions, window, out, spans, span_keys)
        return True


def _split_tiles(self, step, big_rows: int, small_rows: int):
    """(tiles of requests that bring more than `small_rows` rows, cut into `big_rows` rows; one tile for each of the other
    requests), each int32 [n, 3] = (request, first row, rows) on the device, or None. Kept on the step."""
    key = ("split_tiles", big_rows, small_rows)
    if key not in step.host:
        starts = step.host["row_start"]
        big, small = [], []
        for b in range(step.n_requests):
            n = starts[b + 1] - starts[b]
            if n <= small_rows:
                small.append((b, starts[b], n))
            else:
                big += [(b, r0, min(big_rows, starts[b + 1] - r0)) for r0 in range(starts[b], starts[b + 1], big_rows)]
        both = torch.tensor(big + small, dtype=torch.int32).reshape(-1, 3).to(self.device, non_blocking=True)
        step.host[key] = (both[:len(big)] if big else None, both[len(big):] if small else None,
                          max((t[2] for t in small), default=0))
    return step.host[key]


def _prompt_attention(self, q, cache, table, step, scale, window, out, runtime) -> bool:
    """A step with prompt portions. Requests that bring many rows go to the tcgen05 kernel in tiles of 128 M rows (128 / G
    query rows), two CTAs an SM; requests that bring a row or a few (the decode rows of a mixed step) go to the mma.sync
    kernel's form for small tiles, which splits each key tile among its warps. Both cut the keys into the same spans, so
    one join serves the step; the keys are split only when the tiles alone would leave half of the GPU idle."""
    R, Hq, D = q.shape
    Hk = cache.k.shape[1]
    G = Hq // Hk
    tile_rows = lib().tl_attention_tc_tile_rows(Hq, Hk)
    big, small, small_max = self._split_tiles(step, tile_rows, 16 // G)
    n_big = 0 if big is None else big.shape[0]
    n_small = 0 if small is None else small.shape[0]
    ctas, slots = (n_big + n_small) * Hk, 2 * self.sm_count
    span_keys, spans = 0, 1
    if step.max_context > 1024 and 2 * ctas <= slots:
        # (only then: the join reads and writes every row's partial results, which for a prompt's many rows costs as
        # much as the attention of a short context itself)
        want = slots // ctas                                           # spans that fill the GPU once
        span_keys = max(1024, -(-(-(-step.max_context // want)) // 128) * 128)
        spans = -(-step.max_context // span_keys)
        if spans <= 1:
            span_keys, spans = 0, 1
    scratch = runtime.scratch("attention", ops.attention_scratch_floats(R, Hq, D, spans)) if span_keys else None
    common = (step.positions.data_ptr(), float(scale), int(window or 0), out.data_ptr(), ops.ptr(scratch), R, Hq, Hk, D, spans,
              span_keys, self.status.data_ptr(), ops.stream())
    head = (q.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(), table.data_ptr(), table.shape[1], cache.page_size,
            cache.k.shape[0])
    if n_big:
        _check(lib().tl_paged_attention_tc(*head, big.data_ptr(), n_big, min(tile_rows, step.max_rows_per_request), *common),
               "attention_tc")
    if n_small:
        _check(lib().tl_paged_attention_mma(*head, small.data_ptr(), n_small, small_max, *common), "attention_mma")
    if span_keys:
        ops.attention_join(scratch, step.positions, window, out, spans, span_keys)
    return True


TensorCore._split_tiles = _split_tiles
TensorCore._prompt_attention = _prompt_attention


def enable(runtime) -> TensorCore:
    """Build and load the tensor-core library and give `runtime` its kernels: the runtime's bfloat16 products,
    expert feed-forwards and attention go through them from now on."""
    lib()
    runtime.tensorcore = TensorCore(runtime.device, runtime.status)
    runtime.attention_kernels = runtime.tensorcore
    return runtime.tensorcore
