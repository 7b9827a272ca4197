"""The tcgen05 / TMA matrix-product kernels alone against torch in 32-bit: both orientations, every token-tile
size, tails in every dimension, bias, 32-bit and bfloat16 outputs, split-K, and the grouped expert form with the
SwiGLU epilogue against a loop over experts."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def tc():
    from tandemllm_b200.kernels import tensorcore
    from tandemllm_b200.parts import Runtime
    rt = Runtime(torch.device(DEV), torch.bfloat16)
    return tensorcore.enable(rt), rt


def rnd(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(torch.bfloat16)


def rel(got, want):
    return float((got.float().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("M", [1, 8, 17, 64, 100, 128, 129, 300, 1000])
@pytest.mark.parametrize("N,K", [(128, 64), (200, 200), (3072, 2048), (72, 136)])
def test_linear_all_shapes(M, N, K):
    impl, rt = tc()
    x, w, b = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=0.1), torch.randn(N, generator=torch.Generator().manual_seed(3))
    want = x.float() @ w.float().T
    for out_dtype, bias in ((torch.bfloat16, None), (torch.float32, b)):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        assert impl.linear(x.to(DEV), w.to(DEV), None if bias is None else bias.to(DEV), out)
        torch.cuda.synchronize()
        assert int(rt.status) == 0
        ref = want + (0 if bias is None else bias)
        assert rel(out, ref) < (1e-2 if out_dtype == torch.bfloat16 else 1e-4), (M, N, K, out_dtype)


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16, 23, 32])
@pytest.mark.parametrize("N,K", [(128, 64), (200, 200), (72, 136), (2048, 2048), (100, 40), (17, 8), (4096, 1024)])
def test_few_tokens_through_registers_alone(M, N, K):
    """The decode-step product that loads both operands straight into mma.sync registers: every count of token
    tiles, widths with tails in rows and in k (a last chunk of 8, 16 or 24 elements), bias, both output types,
    strided token rows; run twice, the same bits."""
    from tandemllm_b200.kernels import ops, tensorcore
    impl, rt = tc()
    lib = tensorcore.lib()
    xw = rnd(M, K + 8, seed=21).to(DEV)
    x = xw[:, :K]                                                   # row stride K + 8
    w, b = rnd(N, K, seed=22, scale=0.1), torch.randn(N, generator=torch.Generator().manual_seed(23))
    assert lib.tl_gemm_skinny_supported(M, N, K, x.stride(0), K)
    want = x.float().cpu() @ w.float().T
    wd, bd = w.to(DEV), b.to(DEV)
    for out_dtype, bias in ((torch.bfloat16, None), (torch.float32, bd)):
        outs = []
        for _ in range(2):
            out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
            assert lib.tl_gemm_skinny_mma(x.data_ptr(), x.stride(0), wd.data_ptr(), K, ops.ptr(bias), out.data_ptr(), N,
                                          M, N, K, ops.dtype_code(out_dtype), ops.stream()) == 0
            outs.append(out)
        torch.cuda.synchronize()
        assert torch.equal(outs[0], outs[1])
        ref = want + (0 if bias is None else b)
        assert rel(outs[0], ref) < (1e-2 if out_dtype == torch.bfloat16 else 1e-4), (M, N, K, out_dtype)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    assert impl.linear(x, wd, None, out) is True and impl._workspace is None, "linear() takes this kernel for such shapes"
    assert not lib.tl_gemm_skinny_supported(33, N, K, K, K) and not lib.tl_gemm_skinny_supported(M, N, K + 4, K + 4, K + 4)


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("H,K,taps,use_bias", [(200, 136, 3, False), (96, 64, 4, True), (64, 2048, 2, False),
                                               (300, 520, 7, True), (2048, 2048, 3, False)])
def test_in_projection_and_short_conv_in_one_kernel(M, H, K, taps, use_bias):
    """A decode step's in-projection with the convolution and the state's shift in its epilogue: the same bits as the
    projection into bfloat16 followed by the convolution's own decode kernel; channel counts with a tail in the CTA's
    eight, k with a short last chunk, sequences at their first positions beside later ones, a state left alone."""
    from tandemllm_b200.kernels import ops
    impl, rt = tc()
    dev = lambda t: None if t is None else t.to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    x, w = dev(rnd(M, K, seed=40)), dev(rnd(3 * H, K, seed=41, scale=0.1))
    b_in = dev(torch.randn(3 * H, generator=torch.Generator().manual_seed(42))) if use_bias else None
    b_taps = dev(torch.randn(H, generator=torch.Generator().manual_seed(43))) if use_bias else None
    tw = dev(torch.randn(H, taps, generator=torch.Generator().manual_seed(44)))
    state = torch.randn(9, taps - 1, H, generator=torch.Generator().manual_seed(45))
    starts, slots = [0, 1, 2, 5, 40, 3, 0, 9][:M], [2, 0, 3, 4, 6, 8, 1, 5][:M]
    rows = i32(list(range(M)))
    # the two kernels
    bcx = torch.empty(M, 3 * H, dtype=torch.bfloat16, device=DEV)
    assert impl.linear(x, w, b_in, bcx) is True
    st_two, y_two = dev(state.clone()), torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
    ops.short_conv_decode(bcx, tw, b_taps, st_two, i32(slots), rows, i32(starts), y_two)
    # the one
    st, y = dev(state.clone()), torch.full((M, H), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert impl.in_proj_conv(x, w, b_in, tw, b_taps, st, i32(slots), rows, i32(starts), y)
    kept, y_kept = dev(state.clone()), torch.empty_like(y)
    assert impl.in_proj_conv(x, w, b_in, tw, b_taps, kept, i32(slots), rows, i32(starts), y_kept, write_state=False)
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    assert torch.equal(y, y_two) and torch.equal(st, st_two)
    assert torch.equal(y_kept, y_two) and torch.equal(kept.cpu(), state)
    # and the plain formula: bx = B x, y = C (bias + sum_j taps[j] bx[pos - (taps - 1) + j]), inputs before position 0 zero
    z = x.float().cpu() @ w.float().cpu().T + (0 if b_in is None else b_in.cpu())
    assert rel(bcx, z) < 1e-2
    z = bcx.float().cpu()                       # (the projection as it was rounded, so that the state compares exactly)
    B, C, X = z[:, :H], z[:, H:2 * H], z[:, 2 * H:]
    for m in range(M):
        hist = torch.cat([state[slots[m]], (B[m] * X[m])[None]])            # the last `taps` inputs, oldest first
        for j in range(taps):
            if starts[m] - (taps - 1 - j) < 0:
                hist[j] = 0
        conv = (tw.cpu().T * hist).sum(0) + (0 if b_taps is None else b_taps.cpu())
        assert rel(y[m], C[m] * conv) < 1e-2, m
        assert torch.allclose(st[slots[m]].cpu(), hist[1:], atol=1e-6), m
    assert not impl.in_proj_conv(dev(rnd(9, K, seed=46)), w, b_in, tw, b_taps, st, i32(list(range(9))), i32(list(range(9))),
                                 i32([1] * 9), torch.empty(9, H, dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("swap,bn", [(True, 16), (True, 32), (True, 64), (True, 128), (True, 256), (False, 16),
                                     (False, 64), (False, 128), (False, 256)])
def test_every_tile_shape_in_both_orientations(swap, bn):
    impl, rt = tc()
    M, N, K = 150, 330, 520
    x, w = rnd(M, K, seed=4), rnd(N, K, seed=5, scale=0.1)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    impl.gemm(x.to(DEV), w.to(DEV), None, out, swap=swap, bn=bn)
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    assert rel(out, x.float() @ w.float().T) < 1e-3


@pytest.mark.parametrize("act", ["gelu", "relu2", "identity"])
def test_dense_gate_up_with_other_gate_activations(act):
    from tandemllm_b200.kernels import ops
    from tests.test_gpu_kernels import plain_activation
    impl, rt = tc()
    M, H, I = 300, 136, 200
    x, w = rnd(M, H, seed=30), rnd(2 * I, H, seed=31, scale=0.2)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert impl.gated(x.to(DEV), w.to(DEV), out, ops.activation_code(act))
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    g, u = x.float() @ w[:I].float().T, x.float() @ w[I:].float().T
    assert rel(out, plain_activation(act, g) * u) < 1e-2


@pytest.mark.parametrize("M,H,I", [(300, 136, 200), (129, 64, 72), (2048, 256, 640)])
def test_dense_gate_up_with_the_swiglu_epilogue(M, H, I):
    """A prompt's dense feed-forward: gate, up and silu(gate) * up in the persistent kernel (gate and up rows of the
    same outputs stacked into one operand), tails in every dimension; a decode step's few rows are left to the caller."""
    impl, rt = tc()
    x, w = rnd(M, H, seed=30), rnd(2 * I, H, seed=31, scale=0.2)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert impl.gated(x.to(DEV), w.to(DEV), out)
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    g, u = x.float() @ w[:I].float().T, x.float() @ w[I:].float().T
    assert rel(out, torch.nn.functional.silu(g) * u) < 1e-2
    assert not impl.gated(x[:8].to(DEV), w.to(DEV), out[:8])


def test_a_pipeline_wait_that_runs_out_returns_and_leaves_the_gpu_as_it_was():
    """Every mbarrier wait of the tensor-core kernels is bounded. Here one runs out on purpose, without any fault: the
    producer is told to leave one k-block's copies out (a test hook of the launcher), so the MMA issuer waits for a
    barrier that nothing completes. With the bound lowered the wait gives up after a few thousand polls: the kernel
    records status 11, stores nothing, waits for the copies it did start, frees its tensor memory and returns by itself;
    the same product launched again right after is correct."""
    import ctypes

    from tandemllm_b200.kernels import tensorcore
    impl, rt = tc()
    lib = tensorcore.lib()
    lib.tl_tc_set_wait_limit.argtypes, lib.tl_tc_set_wait_limit.restype = [ctypes.c_uint], ctypes.c_int
    lib.tl_tc_test_skip_k_block.argtypes, lib.tl_tc_test_skip_k_block.restype = [ctypes.c_int], None
    M, N, K = 40, 128, 256                       # one CTA of the swapped kernel, four k-blocks, no split
    x, w = rnd(M, K, seed=40).to(DEV), rnd(N, K, seed=41, scale=0.1).to(DEV)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    try:
        assert lib.tl_tc_set_wait_limit(4096) == 0
        lib.tl_tc_test_skip_k_block(2)
        impl.gemm(x, w, None, out)
        torch.cuda.synchronize()                 # returns: the kernel ended by its own bound
        assert int(rt.status) == 11
        assert bool(torch.isnan(out).all()), "a product that gave up must store nothing"
    finally:
        lib.tl_tc_test_skip_k_block(-1)
        assert lib.tl_tc_set_wait_limit(0) == 0
    rt.status.zero_()
    impl.gemm(x, w, None, out)
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    assert rel(out, x.float().cpu() @ w.float().cpu().T) < 1e-3


def test_split_k_is_used_and_repeatable():
    impl, rt = tc()
    M, N, K = 8, 256, 4096                      # 2 CTAs without a split: the k range is cut
    x, w = rnd(M, K, seed=6), rnd(N, K, seed=7, scale=0.05)
    b = torch.randn(N, generator=torch.Generator().manual_seed(8))
    outs = []
    for _ in range(2):
        out = torch.empty(M, N, dtype=torch.float32, device=DEV)
        impl.gemm(x.to(DEV), w.to(DEV), b.to(DEV), out)
        outs.append(out.clone())
    assert impl._workspace is not None
    assert torch.equal(outs[0], outs[1])
    assert rel(outs[0], x.float() @ w.float().T + b) < 1e-3


@pytest.mark.parametrize("R,E,k,H,I", [(4, 8, 2, 128, 64), (8, 32, 4, 256, 192), (64, 8, 3, 136, 72), (700, 6, 2, 128, 96),
                                       (1, 32, 4, 256, 1024), (2, 16, 3, 200, 520), (5, 6, 2, 136, 72),
                                       (8, 4, 4, 72, 40), (7, 3, 3, 88, 24), (8, 2, 2, 72, 40),     # every expert holds every row
                                       (16, 4, 2, 72, 40), (13, 3, 3, 88, 24), (16, 32, 4, 256, 192),  # experts with two tiles of 8
                                       (12, 5, 1, 72, 40), (16, 2, 1, 72, 40), (9, 1, 1, 72, 40),   # top-1: up to 16 pairs, yet an expert with more than 8 rows
                                       (2048, 4, 2, 64, 128)])
def test_grouped_experts_with_swiglu(R, E, k, H, I):
    grouped_experts(R, E, k, H, I, "silu", "sigmoid")


@pytest.mark.parametrize("act,scoring", [("gelu", "softmax"), ("relu2", "sigmoid"), ("identity", "softmax")])
@pytest.mark.parametrize("R,E,k,H,I", [(4, 8, 2, 128, 64), (16, 32, 4, 256, 192), (64, 8, 3, 136, 72), (700, 6, 2, 128, 96)])
def test_grouped_experts_with_other_activations_and_scoring(R, E, k, H, I, act, scoring):
    """The fused expert kernels (the register-only grouped form, the swapped and the persistent tcgen05 forms) with the gate
    activation and the router's scoring function a feed-forward other than LFM2's would name."""
    grouped_experts(R, E, k, H, I, act, scoring)


def _drawn_expert_shapes():
    import random
    rng = random.Random(5)
    shapes = []
    for _ in range(36):
        E = rng.choice([1, 2, 3, 5, 8, 9, 16, 33, 40, 70])
        k = rng.randint(1, min(E, 8))
        R = rng.choice([1, 2, 3, 7, 8, 9, 12, 15, 16, 17, 24, 31, 32, 33, 47, 64, 65, 100, 128, 129, 200, 300])
        shapes.append((R, E, k, rng.choice([72, 136]), rng.choice([40, 72])))
    return shapes


@pytest.mark.parametrize("R,E,k,H,I", _drawn_expert_shapes())
def test_grouped_experts_at_drawn_rows_experts_and_top_k(R, E, k, H, I):
    """The experts' dispatch picks a kernel form by the step's rows, the pairs and the experts (no plan, plan tiles of 8,
    fetched rows, the swapped tile widths, the persistent kernel): drawn combinations around every threshold."""
    grouped_experts(R, E, k, H, I, "silu", "sigmoid")


def grouped_experts(R, E, k, H, I, act, scoring):
    from tandemllm_b200.config import PartSpec
    from tandemllm_b200.parts import make_part
    from tests.test_gpu_kernels import plain_activation
    impl, rt = tc()
    spec = PartSpec("sigmoid_topk_experts", {"num_experts": E, "top_k": k, "intermediate_size": I, "expert_bias": False,
                                             "normalize": True, "scale": 1.0, "activation": act, "scoring": scoring,
                                             "names": {"router": "gate", "bias": "expert_bias", "experts": "experts",
                                                       "gate": "w1", "up": "w3", "down": "w2"}})
    part = make_part("feed_forward", spec, prefix="m.", hidden_size=H)
    W = {"m.gate.weight": rnd(E, H, seed=9, scale=0.5).float()}
    w13, w2 = rnd(E, 2 * I, H, seed=10, scale=0.2), rnd(E, H, I, seed=11, scale=0.2)
    for e in range(E):
        W[f"m.experts.{e}.w1.weight"], W[f"m.experts.{e}.w3.weight"] = w13[e, :I], w13[e, I:]
        W[f"m.experts.{e}.w2.weight"] = w2[e]
    part.weight_specs(set(W))
    part.bind(lambda n: W[n], rt)
    x = rnd(R, H, seed=12)
    ids, wts = part.route(x.float().to(DEV))
    score = x.float() @ W["m.gate.weight"].T
    score = torch.softmax(score, -1) if scoring == "softmax" else torch.sigmoid(score)
    want_ids = torch.sort(score, dim=-1, descending=True, stable=True).indices[:, :k]
    assert torch.equal(ids.cpu().long(), want_ids)
    from tandemllm_b200.kernels import ops
    result = impl.experts(part, x.to(DEV), ids, wts)
    assert result is not None
    out = result.materialize()
    # with the experts' load counted a small step builds a routing plan, without it needs none: the same bits
    part.load = torch.zeros(E, dtype=torch.int64, device=DEV)
    counted = impl.experts(part, x.to(DEV), ids, wts).materialize()
    assert torch.equal(part.load.cpu(), torch.bincount(ids.cpu().flatten().long(), minlength=E))
    assert torch.equal(counted, out)
    part.load = None
    # the same rows as the norm kernel adds them (partial sums of a split down product included)
    residual = torch.zeros(R, H, dtype=torch.float32, device=DEV)
    ops.add_rmsnorm(residual, result, torch.ones(H, device=DEV), 1e-5, torch.empty(R, H, dtype=torch.bfloat16, device=DEV))
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    assert (residual - out).abs().max() <= 1e-5 * out.abs().max()
    want = torch.zeros(R, H)
    xf, idc, wc = x.float(), ids.cpu(), wts.cpu()
    for e in range(E):
        rows, slot = torch.where(idc == e)
        if rows.numel():
            h = plain_activation(act, xf[rows] @ w13[e, :I].float().T) * (xf[rows] @ w13[e, I:].float().T)
            want.index_add_(0, rows, (h.to(torch.bfloat16).float() @ w2[e].float().T) * wc[rows, slot, None])
    assert rel(out, want) < 2e-2


@pytest.mark.parametrize("R,E,k", [(8, 40, 6), (8, 9, 6), (7, 300, 32), (3, 33, 32)])
def test_experts_of_a_small_step_without_a_plan_at_every_count_of_pairs(R, E, k, monkeypatch):
    """The form in which the products' CTAs find each expert's pairs in the ids themselves is used for a few pairs only;
    it takes up to 256 (pairs in several warps of the CTA that looks for them): the same bits as with a plan."""
    from tandemllm_b200.config import PartSpec
    from tandemllm_b200.kernels import tensorcore
    from tandemllm_b200.parts import make_part
    H, I = 72, 40
    outs = []
    for cap in (256, 0):
        monkeypatch.setattr(tensorcore, "SKINNY_PAIRS", cap)
        impl, rt = tc()
        spec = PartSpec("sigmoid_topk_experts", {"num_experts": E, "top_k": k, "intermediate_size": I, "expert_bias": False,
                                                 "normalize": True, "scale": 1.0,
                                                 "names": {"router": "gate", "bias": "expert_bias", "experts": "experts",
                                                           "gate": "w1", "up": "w3", "down": "w2"}})
        part = make_part("feed_forward", spec, prefix="m.", hidden_size=H)
        W = {"m.gate.weight": rnd(E, H, seed=9, scale=0.5).float()}
        w13, w2 = rnd(E, 2 * I, H, seed=10, scale=0.2), rnd(E, H, I, seed=11, scale=0.2)
        for e in range(E):
            W[f"m.experts.{e}.w1.weight"], W[f"m.experts.{e}.w3.weight"] = w13[e, :I], w13[e, I:]
            W[f"m.experts.{e}.w2.weight"] = w2[e]
        part.weight_specs(set(W))
        part.bind(lambda n: W[n], rt)
        x = rnd(R, H, seed=12).to(DEV)
        ids, wts = part.route(x.float())
        result = impl.experts(part, x, ids, wts)
        assert (result.pos_of_pair is impl._pair_order) == (cap > 0)
        outs.append(result.materialize())
        torch.cuda.synchronize()
        assert int(rt.status) == 0
    assert torch.equal(outs[0], outs[1])
    want = torch.zeros(R, H)
    xf, idc, wc = x.float().cpu(), ids.cpu(), wts.cpu()
    for e in range(E):
        rows, slot = torch.where(idc == e)
        if rows.numel():
            h = torch.nn.functional.silu(xf[rows] @ w13[e, :I].float().T) * (xf[rows] @ w13[e, I:].float().T)
            want.index_add_(0, rows, (h.to(torch.bfloat16).float() @ w2[e].float().T) * wc[rows, slot, None])
    assert rel(outs[0], want) < 2e-2


@pytest.mark.parametrize("split", [0, 256, 512])
@pytest.mark.parametrize("Hq,Hk,D,page,window", [(8, 2, 64, 16, None), (4, 4, 64, 16, None), (6, 2, 128, 32, None),
                                                 (8, 1, 64, 16, 100), (32, 8, 64, 16, None), (3, 1, 64, 64, None),
                                                 (5, 1, 128, 16, 300), (8, 2, 64, 128, None), (4, 1, 128, 128, 200),
                                                 (4, 2, 64, 48, None)])
def test_attention_on_tensor_cores(split, Hq, Hk, D, page, window):
    """Prompt portions of several lengths, a sequence's first rows and decode rows at short and long contexts in
    one call, unsplit and split over key spans, against whole-sequence attention."""
    attention_against_plain([700, 90, 7, 300, 513], [1, 23, 7, 150, 1], split, Hq, Hk, D, page, window)


@pytest.mark.parametrize("split", [0, 64, 256])
@pytest.mark.parametrize("Hq,Hk,D,page,window,news", [
    (8, 2, 64, 16, None, [1, 1, 1, 1, 1, 1, 1]), (32, 8, 64, 16, None, [1, 1, 1, 1, 1, 1, 1]),
    (16, 1, 64, 16, 100, [1, 1, 1, 1, 1, 1, 1]), (6, 2, 128, 32, None, [1, 1, 1, 1, 1, 1, 1]),
    (8, 2, 64, 24, 70, [4, 2, 3, 1, 4, 1, 2]), (3, 3, 128, 16, None, [16, 5, 7, 1, 9, 2, 16]),
    (5, 1, 64, 64, 300, [3, 1, 2, 3, 1, 1, 3]), (8, 2, 64, 128, None, [1, 1, 1, 1, 1, 1, 1]),
    (4, 1, 128, 256, 150, [1, 2, 1, 3, 1, 1, 4]), (16, 4, 64, 32, 500, [1, 1, 1, 1, 1, 1, 1])])
def test_attention_of_small_tiles_splits_the_keys_among_warps(split, Hq, Hk, D, page, window, news):
    """Tiles whose rows and heads fit 16 M rows (decoding, and portions of a few rows) run the kernel form in which
    each warp takes a quarter of every key tile: contexts that end inside a warp's quarter, at a tile's edge, a
    sequence's first rows, page sizes that are no power of two."""
    attention_against_plain([700, 90, 16, 300, 513, 64, 65], news, split, Hq, Hk, D, page, window)


@pytest.mark.parametrize("split", [0, 256, 512])
@pytest.mark.parametrize("Hq,Hk,page,window", [(8, 2, 16, None), (4, 4, 16, None), (8, 1, 16, 100), (32, 8, 16, None),
                                               (3, 1, 64, None), (8, 2, 128, None), (4, 1, 128, 200), (6, 2, 8, 300),
                                               (16, 4, 32, None), (5, 1, 256, None), (7, 7, 16, 130)])
def test_prompt_attention_on_tcgen05(split, Hq, Hk, page, window):
    """The tcgen05 kernel (scores and values in tensor memory, tiles of 128 M rows and 128 keys): prompt portions of
    several lengths, a sequence's first rows, portions that end at a tile's edge and decode rows at short and long
    contexts in one call, unsplit and split over key spans, group sizes that do not divide 128, pages of 8 to 256."""
    attention_against_plain([700, 90, 7, 300, 513, 128, 256], [1, 23, 7, 150, 1, 128, 129], split, Hq, Hk, 64, page, window,
                            kernel="tc")


@pytest.mark.parametrize("rows,context", [(2048, 2048), (512, 4096), (1000, 1000)])
def test_prompt_attention_on_tcgen05_over_many_key_tiles(rows, context):
    """Whole prompts and a portion at the end of a long context: a tile walks up to 32 key tiles, the ring of key and
    value slots turns many times, and the running maximum and the rescaling of O are exercised over long rows."""
    attention_against_plain([context], [rows], 0, 32, 8, 64, 16, None, kernel="tc")
    attention_against_plain([context], [rows], 1024, 8, 2, 64, 16, 600, kernel="tc")


@pytest.mark.parametrize("Hq,Hk,window", [(32, 8, None), (8, 2, 900), (4, 4, None)])
def test_a_mixed_step_sends_portions_and_decode_rows_to_their_kernels_over_the_same_spans(Hq, Hk, window):
    """What the dispatcher does for a step with prompt portions: long portions on the tcgen05 kernel, single decode rows
    and portions of a few rows on the mma.sync kernel's small-tile form, both over the same key spans (contexts of
    thousands of keys), one join."""
    import types

    from tests.test_gpu_kernels import paged_setup, plain_attention
    impl, rt = tc()
    D, page = 64, 16
    seqs, news = [3000, 2000, 5000, 90, 4100, 130], [1, 300, 2, 40, 1, 130]
    kc, vc, table, ks, vs = paged_setup(seqs, Hk, D, page, torch.bfloat16, seed=80)
    R = sum(news)
    q = rnd(R, Hq, D, seed=81)
    positions = sum((list(range(L - n, L)) for L, n in zip(seqs, news)), [])
    starts = [0]
    for n in news:
        starts.append(starts[-1] + n)
    step = types.SimpleNamespace(n_requests=len(seqs), max_rows_per_request=max(news), max_context=max(seqs),
                                 positions=torch.tensor(positions, dtype=torch.int32, device=DEV), host={"row_start": starts})
    cache = types.SimpleNamespace(k=kc.to(DEV), v=vc.to(DEV), page_size=page)
    out = torch.full((R, Hq, D), float("nan"), dtype=torch.bfloat16, device=DEV)
    scale = 0.9 / D ** 0.5
    assert impl.attention(q.to(DEV), cache, table.to(DEV), step, scale, window, out, rt)
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    big, small, small_max = impl._split_tiles(step, 128 // (Hq // Hk), 16 // (Hq // Hk))
    assert big is not None and small is not None and int(small[:, 2].max()) == small_max <= 16 // (Hq // Hk)
    at = 0
    for b, (L, n) in enumerate(zip(seqs, news)):
        want = plain_attention(q[at:at + n].float(), ks[b], vs[b], scale, window)
        assert rel(out[at:at + n], want) < 2e-2, f"sequence {b}"
        at += n


def attention_against_plain(seqs, news, split, Hq, Hk, D, page, window, kernel="mma"):
    if kernel == "tc":
        # both forms of the tcgen05 kernel: P back in tensor memory (the default), and P through shared memory
        from tandemllm_b200.kernels import tensorcore
        lib = tensorcore.lib()
        try:
            for p_in_tmem in (0, 1):
                lib.tl_attention_tc_p_in_tensor_memory(p_in_tmem)
                attention_against_plain(seqs, news, split, Hq, Hk, D, page, window, kernel="tc, as set")
        finally:
            lib.tl_attention_tc_p_in_tensor_memory(1)
        return
    kernel = kernel.split(",")[0]
    import types

    from tandemllm_b200.kernels import ops, tensorcore
    from tests.test_gpu_kernels import paged_setup, plain_attention
    impl, rt = tc()
    kc, vc, table, ks, vs = paged_setup(seqs, Hk, D, page, torch.bfloat16, seed=60)
    R = sum(news)
    q = rnd(R, Hq, D, seed=61)
    positions = sum((list(range(L - n, L)) for L, n in zip(seqs, news)), [])
    starts = [0]
    for n in news:
        starts.append(starts[-1] + n)
    pos_dev = torch.tensor(positions, dtype=torch.int32, device=DEV)
    step = types.SimpleNamespace(n_requests=len(seqs), max_rows_per_request=max(news), max_context=max(seqs),
                                 positions=pos_dev, host={"row_start": starts})
    lib = tensorcore.lib()
    if kernel == "tc":
        assert lib.tl_attention_tc_supported(Hq, Hk, D, page)
    tile_rows = lib.tl_attention_tc_tile_rows(Hq, Hk) if kernel == "tc" else lib.tl_attention_mma_tile_rows(Hq, Hk)
    launch = lib.tl_paged_attention_tc if kernel == "tc" else lib.tl_paged_attention_mma
    tiles = impl.query_tiles(step, tile_rows)
    assert int(tiles[:, 2].sum()) == R and int(tiles[:, 2].max()) <= tile_rows
    spans = -(-max(seqs) // split) if split else 1          # `split`: key positions per span, 0 for one pass
    scratch = torch.full((ops.attention_scratch_floats(R, Hq, D, spans),), float("nan"), device=DEV) if split else None
    out = torch.full((R, Hq, D), float("nan"), dtype=torch.bfloat16, device=DEV)
    scale = 0.9 / D ** 0.5
    qd, kd, vd, td = q.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV)      # kept alive until the kernel has run
    code = launch(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), td.data_ptr(),
                  table.shape[1], page, kd.shape[0], tiles.data_ptr(), tiles.shape[0], int(tiles[:, 2].max()),
                  pos_dev.data_ptr(), scale,
                  window or 0, out.data_ptr(), ops.ptr(scratch), R, Hq, Hk, D, spans, int(split),
                  rt.status.data_ptr(), ops.stream())
    assert code == 0, lib.tl_tc_last_error().decode()
    if split:
        ops.attention_join(scratch, pos_dev, window, out, spans, split)
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    at = 0
    for b, (L, n) in enumerate(zip(seqs, news)):
        want = plain_attention(q[at:at + n].float(), ks[b], vs[b], scale, window)
        assert rel(out[at:at + n], want) < 2e-2, f"sequence {b}"
        at += n


@pytest.mark.parametrize("split", [0, 256])
@pytest.mark.parametrize("page", [16, 128])
def test_window_edge_on_tcgen05(page, split):
    """The same planted key at the window's edge through the tcgen05 prompt kernel."""
    test_window_edge_on_tensor_cores(64, page, split, 1, kernel="tc")


@pytest.mark.parametrize("use_tma", [1, 0])
@pytest.mark.parametrize("split", [0, 256])
@pytest.mark.parametrize("D,page", [(64, 16), (64, 48), (64, 128), (128, 16), (128, 48), (128, 128)])
def test_window_edge_on_tensor_cores(D, page, split, use_tma, kernel="mma"):
    """The tensor-core kernel's window: with a window of w the key w positions behind a row is out and the one w - 1
    behind it is in. One key is made to match the queries so strongly that the output is its value when it is visible:
    at the first position inside the window of the checked row (in), and one before it (out). A decode row, and a prompt
    portion whose rows straddle that key (visible to its first rows, hidden from its last). Pages wholly behind every
    row's window are gone (-1 in the table), which must not be recorded as a missing page. With and without a split over
    key spans, with the producer warp's TMA copies and with cp.async from every thread."""
    import types

    from tandemllm_b200.kernels import ops, tensorcore
    from tests.test_gpu_kernels import paged_setup, plain_attention
    impl, rt = tc()
    lib = tensorcore.lib()
    Hq, Hk, w = 4, 1, 150
    seqs, news = [700, 420], [1, 40]                     # a decode row at 699; a portion at positions 380..419
    lib.tl_attention_mma_use_tma(use_tma)
    try:
        for which, hot in (("decode, in", 699 - w + 1), ("decode, out", 699 - w), ("portion, straddled", 419 - w + 1 - 20)):
            kc, vc, table, ks, vs = paged_setup(seqs, Hk, D, page, torch.bfloat16, seed=70)
            # every query of a request is one direction plus a little noise, so that one key can match them all
            g = torch.Generator().manual_seed(71)
            base = torch.randn(2, D, generator=g)
            q = torch.cat([(base[bb] + 0.25 * torch.randn(n, Hq, D, generator=g)) for bb, n in enumerate(news)]).to(torch.bfloat16)
            b = 0 if which.startswith("decode") else 1
            key = (6 * base[b] / base[b].norm()).to(torch.bfloat16)
            ks[b][hot] = key.float()
            kc[int(table[b, hot // page]), :, hot % page] = key
            for bb, (L, n) in enumerate(zip(seqs, news)):      # pages that even the portion's first row no longer sees
                table[bb, :max(0, (L - n) - w + 1) // page] = -1
            positions = sum((list(range(L - n, L)) for L, n in zip(seqs, news)), [])
            pos_dev = torch.tensor(positions, dtype=torch.int32, device=DEV)
            step = types.SimpleNamespace(n_requests=2, max_rows_per_request=max(news), max_context=max(seqs),
                                         positions=pos_dev, host={"row_start": [0, 1, 41]})
            tile_rows = lib.tl_attention_tc_tile_rows(Hq, Hk) if kernel == "tc" else lib.tl_attention_mma_tile_rows(Hq, Hk)
            launch = lib.tl_paged_attention_tc if kernel == "tc" else lib.tl_paged_attention_mma
            tiles = impl.query_tiles(step, tile_rows)
            spans = -(-max(seqs) // split) if split else 1
            R = sum(news)
            scratch = torch.full((ops.attention_scratch_floats(R, Hq, D, spans),), float("nan"), device=DEV) if split else None
            out = torch.full((R, Hq, D), float("nan"), dtype=torch.bfloat16, device=DEV)
            qd, kd, vd, td = q.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV)
            code = launch(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), td.data_ptr(), table.shape[1], page,
                          kd.shape[0], tiles.data_ptr(), tiles.shape[0], int(tiles[:, 2].max()),
                          pos_dev.data_ptr(), 1.0, w, out.data_ptr(), ops.ptr(scratch), R, Hq, Hk, D, spans,
                          int(split), rt.status.data_ptr(), ops.stream())
            assert code == 0
            if split:
                ops.attention_join(scratch, pos_dev, w, out, spans, split)
            torch.cuda.synchronize()
            assert int(rt.status) == 0, f"{which}: a page behind the window was asked for"
            at = 0
            for bb, (L, n) in enumerate(zip(seqs, news)):
                want = plain_attention(q[at:at + n].float(), ks[bb], vs[bb], 1.0, w)
                assert rel(out[at:at + n], want) < 2e-2, f"{which}: sequence {bb}"
                at += n
            # the planted key does decide: the rows that see it put most of their weight on it, the others none
            if b == 0:
                sees = which == "decode, in"
                moved = rel(out[:1], vs[0][hot][None].expand(1, Hq, D))
                assert (moved < 0.2) == sees, (which, moved)
            else:
                first, last = out[1], out[40]                  # positions 380 (sees the key) and 419 (does not)
                assert rel(first[None], vs[1][hot][None].expand(1, Hq, D)) < 0.2
                assert rel(last[None], vs[1][hot][None].expand(1, Hq, D)) > 0.5
    finally:
        lib.tl_attention_mma_use_tma(1)


def test_decode_tiles_are_built_on_the_device():
    import types
    impl, rt = tc()
    step = types.SimpleNamespace(n_requests=5, max_rows_per_request=1, host={})
    assert impl.query_tiles(step, 16).tolist() == [[b, b, 1] for b in range(5)]


def test_shapes_tma_cannot_take_fall_back():
    impl, rt = tc()
    x, w = rnd(4, 100, seed=13), rnd(8, 100, seed=14)          # k = 100 is not a multiple of 8
    out = torch.empty(4, 8, dtype=torch.bfloat16, device=DEV)
    assert not impl.linear(x.to(DEV), w.to(DEV), None, out)
    from tandemllm_b200.parts.linear import linear
    got = linear(rt, x.to(DEV), w.to(DEV))
    assert rel(got, x.float() @ w.float().T) < 1e-2


# ---- the product on pairs of SMs (csrc/tc_gemm_pair.cu) ----
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (1, 256, 64), (17, 40, 72), (300, 520, 192), (255, 257, 264), (1000, 136, 520),
                                   (2048, 768, 1024)])
def test_pair_product_at_every_kind_of_tail(M, N, K):
    """Token rows that end a 16-row step of the MMA's N side early, outputs that end a CTA's 128 rows (or the pair's 256)
    early, a k that ends a 64-element block early; bias, both output types; run twice, the same bits."""
    impl, rt = tc()
    x, w = rnd(M, K, seed=61), rnd(N, K, seed=62, scale=0.1)
    b = torch.randn(N, generator=torch.Generator().manual_seed(63))
    want = x.float() @ w.float().T
    for out_dtype, bias in ((torch.bfloat16, None), (torch.float32, b)):
        outs = []
        for _ in range(2):
            out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
            impl.gemm_pair(x.to(DEV), w.to(DEV), None if bias is None else bias.to(DEV), out)
            torch.cuda.synchronize()
            assert int(rt.status) == 0
            outs.append(out)
        assert torch.equal(outs[0], outs[1])
        assert rel(outs[0], want + (0 if bias is None else bias)) < (1e-2 if out_dtype == torch.bfloat16 else 1e-4), (M, N, K)


@pytest.mark.parametrize("M,N,K,runs", [(300, 520, 1000, 4), (512, 2048, 2048, 4), (130, 264, 136, 3), (1000, 136, 520, 2)])
def test_pair_product_in_runs_of_k_blocks_leaves_partial_sums_that_add_up(M, N, K, runs):
    """The reduction cut into runs, each a work item with a partial result of its own ([runs, M, N], 32-bit; the bias in
    the first): the parts add up to the product, a last run shorter than the others and a k that ends a block early
    included; the same bits twice; a run count that would leave a run empty is refused. Through `linear` with `defer`, a
    portion of a few hundred rows comes back as such partial sums and its norm adds them."""
    impl, rt = tc()
    x, w = rnd(M, K, seed=71), rnd(N, K, seed=72, scale=0.1)
    b = torch.randn(N, generator=torch.Generator().manual_seed(73))
    want = x.float() @ w.float().T + b
    outs = []
    for _ in range(2):
        out = torch.full((runs, M, N), float("nan"), dtype=torch.float32, device=DEV)
        impl.gemm_pair(x.to(DEV), w.to(DEV), b.to(DEV), out.view(runs * M, N), rows=M, splits=runs)
        torch.cuda.synchronize()
        assert int(rt.status) == 0
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    total = torch.zeros(M, N, device=DEV)
    for part in outs[0]:
        total += part
    assert rel(total, want) < 1e-4, (M, N, K, runs)
    kb = -(-K // 64)
    if kb >= 3:
        empty = kb - 1 if -(-kb // (kb - 1)) * (kb - 2) >= kb else None       # ceil(kb / runs) * (runs - 1) >= kb: a run is empty
        if empty:
            with pytest.raises(RuntimeError, match="none may be empty"):
                impl.gemm_pair(x.to(DEV), w.to(DEV), None, torch.empty(empty * M, N, device=DEV), rows=M, splits=empty)
    with pytest.raises(RuntimeError, match="runs of k-blocks need"):
        impl.gemm_pair(x.to(DEV), w.to(DEV), None, torch.empty(runs * M, N, dtype=torch.bfloat16, device=DEV), rows=M, splits=runs)


def test_a_deferred_prompt_product_with_few_tiles_comes_back_in_parts_and_the_norm_adds_them():
    from tandemllm_b200.kernels import ops
    impl, rt = tc()
    M, N, K = 512, 2048, 2048
    x, w = rnd(M, K, seed=74).to(DEV), rnd(N, K, seed=75, scale=0.05).to(DEV)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    got = impl.linear(x, w, None, out, defer=True)
    assert isinstance(got, ops.PartialSums) and got.parts > 1
    whole = torch.empty(M, N, dtype=torch.float32, device=DEV)
    impl.gemm_pair(x, w, None, whole)
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    assert rel(got.materialize(), whole.cpu()) < 1e-5
    # the norm kernel adds the parts itself: the same residual and normed rows as from the materialised sum
    res_a = rnd(M, N, seed=76).float().to(DEV)
    res_b = res_a.clone()
    weight = torch.ones(N, device=DEV)
    na = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    nb = torch.empty_like(na)
    ops.add_rmsnorm(res_a, got, weight, 1e-5, na)
    ops.add_rmsnorm(res_b, got.materialize(), weight, 1e-5, nb)
    assert rel(res_a, res_b.cpu()) < 1e-6 and rel(na, nb.float().cpu()) < 1e-2


def test_pair_product_into_a_wider_output_with_strided_token_rows():
    impl, rt = tc()
    M, N, K = 130, 264, 136
    xw = rnd(M, K + 24, seed=64).to(DEV)
    x, w = xw[:, 8:8 + K], rnd(N, K, seed=65, scale=0.1).to(DEV)          # rows 16-byte aligned, stride K + 24
    wide = torch.full((M, N + 40), float("nan"), dtype=torch.bfloat16, device=DEV)
    impl.gemm_pair(x, w, None, wide[:, 8:8 + N])
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    assert rel(wide[:, 8:8 + N], x.float().cpu() @ w.float().cpu().T) < 1e-2
    assert bool(torch.isnan(wide[:, :8]).all()) and bool(torch.isnan(wide[:, 8 + N:]).all())


@pytest.mark.parametrize("act", ["silu", "gelu", "relu2", "identity"])
@pytest.mark.parametrize("M,H,I", [(300, 136, 200), (40, 64, 72), (1024, 256, 640)])
def test_pair_product_with_the_gated_epilogue(M, H, I, act):
    from tandemllm_b200.kernels import ops
    from tests.test_gpu_kernels import plain_activation
    impl, rt = tc()
    x, w = rnd(M, H, seed=66), rnd(2 * I, H, seed=67, scale=0.2)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    impl.gemm_pair(x.to(DEV), w.to(DEV), None, out, gated=ops.activation_code(act), n_out=I)
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    g, u = x.float() @ w[:I].float().T, x.float() @ w[I:].float().T
    assert rel(out, plain_activation(act, g) * u) < 1e-2


@pytest.mark.parametrize("tile", [256, 128, 48])
@pytest.mark.parametrize("R,E,k,H,I", [(64, 8, 4, 128, 256), (700, 32, 4, 256, 264), (512, 5, 2, 136, 72), (1500, 3, 1, 64, 136)])
def test_pair_product_over_a_routing_plan_of_ragged_tiles(R, E, k, H, I, tile):
    """The routed experts' two products over plans of several tile heights: experts with no rows, with a few, with
    more than a tile; every tile's MMAs are as wide as the tile has rows."""
    from tandemllm_b200.kernels import ops
    impl, rt = tc()
    g = torch.Generator().manual_seed(R + E)
    skew = torch.rand(E, generator=g) ** 3 + 1e-3                       # some experts get most of the rows
    ids = torch.stack([torch.multinomial(skew, k, generator=g) for _ in range(R)]).int().to(DEV)
    plan = ops.MoePlan(R * k, E, tile, torch.device(DEV)).build(ids)
    x = rnd(R, H, seed=68).to(DEV)
    order = plan.sorted_pairs[:R * k].long()
    xs = x[order // k].contiguous()
    wgu, wd = rnd(E, 2 * I, H, seed=69, scale=0.1).to(DEV), rnd(E, H, I, seed=70, scale=0.1).to(DEV)
    act = torch.full((R * k, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    impl.gemm_pair(xs, wgu.view(E * 2 * I, H), None, act, rows_per_group=2 * I, plan=plan, gated=1, n_out=I)
    y = torch.full((R * k, H), float("nan"), dtype=torch.float32, device=DEV)
    impl.gemm_pair(act, wd.view(E * H, I), None, y, rows_per_group=H, plan=plan, n_out=H)
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    expert = ids.flatten()[order].long()
    for e in range(E):
        m = expert == e
        if not bool(m.any()):
            continue
        gu = xs[m].float() @ wgu[e].float().T
        want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        assert rel(act[m], want.cpu()) < 1e-2, e
        assert rel(y[m], (act[m].float() @ wd[e].float().T).cpu()) < 1e-3, e


def test_pair_product_refuses_a_plan_of_taller_tiles_than_it_takes():
    from tandemllm_b200.kernels import ops
    impl, rt = tc()
    ids = torch.zeros(600, 1, dtype=torch.int32, device=DEV)
    plan = ops.MoePlan(600, 2, 512, torch.device(DEV)).build(ids)
    x, w = rnd(600, 64, seed=71).to(DEV), rnd(2 * 128, 64, seed=72).to(DEV)
    out = torch.zeros(600, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.KernelError, match="tiles of 512 rows"):
        impl.gemm_pair(x, w, None, out, rows_per_group=128, plan=plan, n_out=128)


@pytest.mark.parametrize("gated", [0, 1])
def test_a_wait_of_the_pair_product_that_runs_out_ends_both_ctas_and_leaves_the_gpu_as_it_was(gated):
    """As for the one-CTA kernels: both producers leave one k-block's copies out, so the MMA issuer of the pair's first
    CTA waits for a barrier that nothing completes. With the bound lowered the wait gives up: status 11, nothing stored,
    each CTA tells the other, the pair meets at its cluster barrier, frees its tensor memory and returns; the same
    product launched again right after is correct."""
    import ctypes

    from tandemllm_b200.kernels import tensorcore
    impl, rt = tc()
    lib = tensorcore.lib()
    lib.tl_tc_pair_set_wait_limit.argtypes, lib.tl_tc_pair_set_wait_limit.restype = [ctypes.c_uint], ctypes.c_int
    lib.tl_tc_pair_test_skip_k_block.argtypes, lib.tl_tc_pair_test_skip_k_block.restype = [ctypes.c_int], None
    M, N, K = 200, 256, 256                      # one pair, one tile, four k-blocks
    x, w = rnd(M, K, seed=73).to(DEV), rnd((2 if gated else 1) * N, K, seed=74, scale=0.1).to(DEV)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    try:
        assert lib.tl_tc_pair_set_wait_limit(4096) == 0
        lib.tl_tc_pair_test_skip_k_block(2)
        impl.gemm_pair(x, w, None, out, gated=gated, n_out=N)
        torch.cuda.synchronize()                 # returns: the kernel ended by its own bound
        assert int(rt.status) == 11
        assert bool(torch.isnan(out).all()), "a product that gave up must store nothing"
    finally:
        lib.tl_tc_pair_test_skip_k_block(-1)
        assert lib.tl_tc_pair_set_wait_limit(0) == 0
    rt.status.zero_()
    impl.gemm_pair(x, w, None, out, gated=gated, n_out=N)
    torch.cuda.synchronize()
    assert int(rt.status) == 0
    xf, wf = x.float().cpu(), w.float().cpu()
    want = torch.nn.functional.silu(xf @ wf[:N].T) * (xf @ wf[N:].T) if gated else xf @ wf.T
    assert rel(out, want) < 1e-3


@pytest.mark.parametrize("which", ["pair", "single"])
def test_prompt_products_through_either_kernel(which, monkeypatch):
    """`gemm` sends the prompt-sized form to the pair kernel or, when told so, to the one-CTA persistent kernel."""
    from tandemllm_b200.kernels import ops, tensorcore
    monkeypatch.setattr(tensorcore, "PROMPT_PRODUCT", which)
    impl, rt = tc()
    M, N, K = 700, 330, 520
    x, w = rnd(M, K, seed=75), rnd(N, K, seed=76, scale=0.1)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    before = ops.launches
    impl.gemm(x.to(DEV), w.to(DEV), None, out, swap=False, bn=256)
    torch.cuda.synchronize()
    assert int(rt.status) == 0 and ops.launches == before + 1
    assert rel(out, x.float() @ w.float().T) < 1e-3
    assert impl.expert_tile(8192, 32)[2] == (256 if which == "pair" else 128)


@pytest.mark.parametrize("gated", [0, 1])
@pytest.mark.parametrize("M,N,K", [(300, 520, 192), (129, 264, 72), (1000, 1792, 256)])
def test_pair_product_with_two_ctas_an_sm(M, N, K, gated):
    """The form with half the shared and tensor memory a CTA (the gated product on tiles of 128 token rows), which a
    routing plan of tiles up to 128 rows selects: the same results as the plain rule, run twice the same bits."""
    impl, rt = tc()
    x, w = rnd(M, K, seed=81), rnd((2 if gated else 1) * N, K, seed=82, scale=0.1)
    outs = []
    for _ in range(2):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        impl.gemm_pair(x.to(DEV), w.to(DEV), None, out, gated=gated, n_out=N, per_sm=2)
        torch.cuda.synchronize()
        assert int(rt.status) == 0
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    full = x.float() @ w.float().T
    want = torch.nn.functional.silu(full[:, :N]) * full[:, N:] if gated else full
    assert rel(outs[0], want) < 1e-2
