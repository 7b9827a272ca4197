"""Each kernel alone against a plain torch reference of the same operation, at sizes other than the tiny
models': widths and vocabularies that are no powers of two, head sizes in steps of 16, odd head counts and
groups, tails shorter than a tile. Where random inputs would hide a fault (a far key among hundreds, a
window's edge, a page's edge) the inputs are made so that it shows.
"""

import math

import pytest
import torch

from tests import plain_lfm2 as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from tandemllm_b200.kernels import ops as o
    o.core()
    return o


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def close(got, want, dtype, what=""):
    got, want = got.float().cpu(), want.float().cpu()
    scale = want.abs().max().clamp_min(1e-6)
    err = float((got - want).abs().max() / scale)
    assert err <= tol(dtype), f"{what}: error {err:.3g} of the largest value"


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


# ------------------------------------------------------------------------------------------ rows
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [200, 96, 2048, 5000])
def test_embed_and_add_rmsnorm(dtype, hidden):
    o = ops()
    V, R = 77, 13
    table = rnd(V, hidden, seed=1).to(dtype)
    toks = torch.randint(0, V, (R,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    res = torch.empty(R, hidden, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.embed_rows(table.to(DEV), toks.to(DEV), res, status)
    assert torch.equal(res.cpu(), table[toks.long()].float()) and int(status) == 0
    w = 1 + rnd(hidden, seed=3, scale=0.2)
    delta = rnd(R, hidden, seed=4)
    eps = 3e-4
    want_res = table[toks.long()].float() + delta
    want = P.rms_norm(want_res, w, eps)
    out = torch.empty(R, hidden, dtype=dtype, device=DEV)
    out32 = torch.empty(R, hidden, dtype=torch.float32, device=DEV)
    o.add_rmsnorm(res, delta.to(DEV), w.to(DEV), eps, out, None, out32)
    close(res, want_res, torch.float32, "residual")
    close(out, want, dtype, "normed")
    close(out32, want, torch.float32, "normed32")
    # gathered rows, residual untouched
    before = res.clone()
    idx = torch.tensor([5, 0, 12], dtype=torch.int32)
    out2 = torch.empty(3, hidden, dtype=dtype, device=DEV)
    o.add_rmsnorm(res, delta.to(DEV), w.to(DEV), eps, out2, idx.to(DEV))
    close(out2, P.rms_norm(want_res[idx.long()] + delta[idx.long()], w, eps), dtype, "gathered")
    assert torch.equal(res, before)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("R", [7, 100])
def test_add_rmsnorm_adds_deferred_branch_outputs_and_routes(dtype, R):
    """The forms a branch output may arrive in (partial sums of a split product; the rows of an expert layer with
    their weights) give what adding the plain tensor gives, and the fused router gives the separate router's choice
    (with many rows a block norms and routes several rows; 100 rows leave a partly filled last block)."""
    o = ops()
    H, S, E, k = 136, 3, 12, 4
    res0, w = rnd(R, H, seed=1), 1 + rnd(H, seed=2, scale=0.2)
    parts = rnd(S, R, H, seed=3)
    want = P.rms_norm(res0 + parts.sum(0), w, 1e-5)
    res = res0.clone().to(DEV)
    out = torch.empty(R, H, dtype=dtype, device=DEV)
    o.add_rmsnorm(res, o.PartialSums(parts.to(DEV).reshape(-1), S, R, H), w.to(DEV), 1e-5, out)
    close(out, want, dtype, "partial sums")
    close(res, res0 + parts.sum(0), torch.float32, "residual after partial sums")
    # expert rows: each row adds its k slots in ascending expert id
    ids = torch.stack([torch.randperm(E, generator=torch.Generator().manual_seed(10 + r))[:k] for r in range(R)]).int()
    wts = torch.rand(R, k, generator=torch.Generator().manual_seed(4))
    y = rnd(R * k, H, seed=5)
    pos = torch.randperm(R * k, generator=torch.Generator().manual_seed(6)).int()
    added = torch.zeros(R, H)
    for r in range(R):
        for j in sorted(range(k), key=lambda j: int(ids[r, j])):
            added[r] += wts[r, j] * y[pos[r * k + j]]
    res = res0.clone().to(DEV)
    rows = o.ExpertRows(y.to(DEV), pos.to(DEV), ids.to(DEV), wts.to(DEV))
    o.add_rmsnorm(res, rows, w.to(DEV), 1e-5, out)
    close(out, P.rms_norm(res0 + added, w, 1e-5), dtype, "expert rows")
    close(rows.materialize(), added, torch.float32, "materialised expert rows")
    # the router inside the norm kernel
    gate, bias = rnd(E, H, seed=7, scale=0.3), rnd(E, seed=8, scale=0.2)
    route = {"weight": gate.to(DEV), "bias": bias.to(DEV), "k": k, "normalize": True, "floor": 1e-6, "scale": 1.5,
             "ids": torch.empty(R, k, dtype=torch.int32, device=DEV), "wts": torch.empty(R, k, dtype=torch.float32, device=DEV)}
    res = res0.clone().to(DEV)
    o.add_rmsnorm(res, None, w.to(DEV), 1e-5, out, None, None, route)
    n32 = P.rms_norm(res0, w, 1e-5)
    cfg = dict(num_experts_per_tok=k, use_expert_bias=True, norm_topk_prob=True, routed_scaling_factor=1.5)
    want_ids, want_w = P.route(n32, {"gate.weight": gate, "expert_bias": bias}, "", cfg)
    assert torch.equal(route["ids"].cpu().long(), want_ids)
    close(route["wts"], want_w, torch.float32, "fused routing weights")
    close(out, n32, dtype, "normed rows beside the router")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,E,k", [(2048, 32, 4), (2048, 64, 4), (136, 12, 3), (4100, 40, 5), (2048, 96, 4)])
def test_the_router_inside_the_norm_routes_a_row_the_same_alone_and_among_many(dtype, H, E, k):
    """A prompt's rows are normed and routed several a block, a decode step's one a block: the same experts must be
    chosen, and the weights and the normed rows may differ by rounding only (the sum of squares of a row is added up by 64
    threads in one form and by 512 in the other), or a row would route differently depending on what else is in its step."""
    o = ops()
    R = 150
    res0, w = rnd(R, H, seed=1), 1 + rnd(H, seed=2, scale=0.2)
    gate, bias = rnd(E, H, seed=7, scale=0.3), rnd(E, seed=8, scale=0.2)

    def run(lo, hi):
        n = hi - lo
        route = {"weight": gate.to(DEV), "bias": bias.to(DEV), "k": k, "normalize": True, "floor": 1e-6, "scale": 1.0,
                 "ids": torch.empty(n, k, dtype=torch.int32, device=DEV), "wts": torch.empty(n, k, dtype=torch.float32, device=DEV)}
        out = torch.empty(n, H, dtype=dtype, device=DEV)
        o.add_rmsnorm(res0[lo:hi].clone().to(DEV), None, w.to(DEV), 1e-5, out, None, None, route)
        return route["ids"].cpu(), route["wts"].cpu(), out.float().cpu()
    many = run(0, R)                                       # more than 64 rows: several rows a block
    few = [run(lo, min(lo + 50, R)) for lo in range(0, R, 50)]      # at most 64: one row a block
    alone = [torch.cat([f[j] for f in few]) for j in range(3)]
    assert torch.equal(many[0], alone[0]), "the chosen experts, in order"
    assert float((many[1] - alone[1]).abs().max()) <= 2e-6, "weights"
    assert float((many[2] - alone[2]).abs().max()) <= (1e-5 if dtype == torch.float32 else 2e-2) * float(alone[2].abs().max())
    # a step of a few rows: a cluster of CTAs a row shares the experts out (from 16 experts on); the same bits as one block a row
    tiny = [run(lo, lo + n) for lo, n in ((0, 11), (11, 1), (12, 16), (28, 5))]
    for j in range(3):
        assert torch.equal(torch.cat([t[j] for t in tiny]), alone[j][:33]), ("a few rows", j)
    # 17 to 37 rows: clusters of four; up to 74 (the runs of 50 above): of two; more, one row a block still: one CTA a row
    mid = [run(0, 30), run(30, 130)]
    for j in range(3):
        assert torch.equal(torch.cat([t[j] for t in mid]), alone[j][:130]), ("clusters of four, one CTA a row", j)
    n32 = P.rms_norm(res0, w, 1e-5)
    cfg = dict(num_experts_per_tok=k, use_expert_bias=True, norm_topk_prob=True, routed_scaling_factor=1.0)
    want_ids, want_w = P.route(n32, {"gate.weight": gate, "expert_bias": bias}, "", cfg)
    assert torch.equal(many[0].long(), want_ids)
    close(many[1], want_w, torch.float32, "routing weights")


@pytest.mark.parametrize("P_rows,E,k", [(8, 32, 4), (64, 6, 3), (256, 32, 4), (257, 32, 4), (1500, 8, 4), (3000, 200, 3), (1025, 1000, 5), (4096, 32, 4),
                                        (6000, 8, 3), (4500, 64, 4)])
def test_plan_forms_agree_and_copy_rows(P_rows, E, k):
    """The one-kernel plan (a decode step or a short portion: up to 1024 pairs), the chunked plan whose blocks count all pairs themselves (up to 16384 pairs)
    and the chunked plan behind a histogram kernel (more; pairs of one expert spread over many chunks and warps) are
    the same stable sort; the one-kernel form also copies the token rows into expert-sorted order."""
    o = ops()
    g = torch.Generator().manual_seed(9)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(P_rows)]).int().to(DEV)
    x = rnd(P_rows, 64, seed=10).to(torch.bfloat16).to(DEV)
    xs = torch.zeros(P_rows * k, 64, dtype=torch.bfloat16, device=DEV)
    plan = o.MoePlan(P_rows * k, E, 16, DEV).build(ids, x, xs)
    flat = ids.cpu().reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    assert torch.equal(plan.sorted_pairs[:P_rows * k].cpu().long(), order)
    assert torch.equal(plan.counts.cpu().long(), torch.bincount(flat, minlength=E))
    assert torch.equal(plan.offsets.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), torch.bincount(flat, minlength=E).cumsum(0)]))
    assert torch.equal(plan.pos_of_pair[:P_rows * k].cpu().long()[order], torch.arange(P_rows * k))
    nt = int(plan.n_tiles)
    assert nt == sum(-(-int(c) // 16) for c in plan.counts.cpu())
    assert sum(int(r) for r in plan.tile_rows[:nt].cpu()) == P_rows * k
    want_tiles = [(e, int(plan.offsets[e]) + t, min(16, int(c) - t)) for e, c in enumerate(plan.counts.cpu().tolist())
                  for t in range(0, int(c), 16)]
    assert list(zip(plan.tile_group[:nt].cpu().tolist(), plan.tile_row0[:nt].cpu().tolist(),
                    plan.tile_rows[:nt].cpu().tolist())) == want_tiles
    groups, row0 = plan.tile_group[:nt].cpu().tolist(), plan.tile_row0[:nt].cpu().tolist()
    assert groups == sorted(groups) and all(int(plan.offsets[g]) <= r < int(plan.offsets[g + 1]) for g, r in zip(groups, row0))
    assert plan.copied == (P_rows * k <= 1024)
    if plan.copied:
        assert torch.equal(xs.cpu(), x.cpu()[order // k])


def test_a_device_graph_replays_what_was_captured_from_a_pool_of_its_own():
    """`ops.DeviceGraph` (runtime-API capture with torch's allocator pointed at a memory pool): tensors made during the
    capture keep their memory, a replay runs the captured kernels on whatever the inputs hold by then, a second graph
    captured into the same pool reuses the memory of tensors dropped since, and a failed capture leaves the stream usable."""
    o = ops()
    pool = torch.cuda.MemPool()
    side = torch.cuda.Stream()
    res = rnd(4, 256, seed=31).to(DEV)
    w = (1 + rnd(256, seed=32, scale=0.1)).to(DEV)
    delta = rnd(4, 256, seed=33).to(DEV)
    torch.cuda.synchronize()

    def capture(body):
        g = o.DeviceGraph()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g.capture_begin(pool)
            try:
                out = body()
            finally:
                g.capture_end()
        torch.cuda.current_stream().wait_stream(side)
        return g, out

    def body():
        work = res.clone()                              # allocated from the pool, written by a captured kernel
        normed = torch.empty(4, 256, dtype=torch.float32, device=DEV)
        o.add_rmsnorm(work, delta, w, 1e-5, normed)
        return normed

    reserved = torch.cuda.memory_reserved()
    g1, out1 = capture(body)
    assert g1.nodes >= 2
    for turn in range(2):
        delta.fill_(float(turn))
        g1.replay()
        torch.cuda.synchronize()
        want = P.rms_norm(res.cpu() + turn, w.cpu(), 1e-5)
        close(out1.cpu(), want, torch.float32, f"replay {turn}")
    grown = torch.cuda.memory_reserved()
    del g1, out1
    g2, out2 = capture(body)
    assert torch.cuda.memory_reserved() == grown >= reserved, "the dropped graph's memory is used again"
    g2.replay()
    torch.cuda.synchronize()
    close(out2.cpu(), P.rms_norm(res.cpu() + 1, w.cpu(), 1e-5), torch.float32, "second graph")
    # another thread's CUDA work in the middle of a capture (an allocation, a copy and its wait) neither fails nor breaks
    # the capture: captures run in thread-local mode, and the pool is the capturing thread's alone
    import threading
    seen = {}

    def elsewhere():
        other = torch.arange(1 << 16, device=DEV, dtype=torch.float32)
        seen["sum"] = float(other.sum().item())

    def body_with_company():
        out = body()
        t = threading.Thread(target=elsewhere)
        t.start()
        t.join()
        return out

    g3, out3 = capture(body_with_company)
    assert seen["sum"] == float(sum(range(1 << 16)))
    g3.replay()
    torch.cuda.synchronize()
    close(out3.cpu(), P.rms_norm(res.cpu() + 1, w.cpu(), 1e-5), torch.float32, "a capture with company")
    with pytest.raises(ZeroDivisionError):
        capture(lambda: 1 // 0)
    assert not torch.cuda.is_current_stream_capturing()
    g2.replay()
    torch.cuda.synchronize()


@pytest.mark.parametrize("R,E,k,tile", [(8, 32, 4, 8), (5, 64, 4, 8), (1, 32, 4, 8), (3, 200, 5, 8), (8, 12, 4, 2), (2, 1000, 16, 8),
                                        (16, 7, 2, 3), (1, 1, 1, 8), (16, 32, 4, 8), (11, 64, 4, 8), (9, 300, 7, 8), (33, 5, 1, 4)])
def test_the_one_warp_plan_of_a_small_step_equals_the_others(R, E, k, tile):
    """Up to 64 pairs and no rows to copy: one warp builds the plan, a pair or two a lane, the experts 32 at a time. Field by
    field what the one-kernel form writes for the same ids, and a stable sort by expert."""
    o = ops()
    g = torch.Generator().manual_seed(14)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(R)]).int().to(DEV)
    P = R * k
    assert P <= 64
    warp = o.MoePlan(P, E, tile, DEV)
    for t in (warp.counts, warp.offsets, warp.sorted_pairs, warp.pos_of_pair, warp.tile_group, warp.tile_row0, warp.tile_rows, warp.n_tiles):
        t.fill_(-3)
    warp.build(ids)
    x = rnd(R, 64, seed=15).to(torch.bfloat16).to(DEV)
    other = o.MoePlan(P, E, tile, DEV).build(ids, x, torch.zeros(P, 64, dtype=torch.bfloat16, device=DEV))
    assert other.copied and not warp.copied
    flat = ids.cpu().reshape(-1).long()
    assert torch.equal(warp.sorted_pairs[:P].cpu().long(), torch.sort(flat, stable=True).indices)
    nt = int(other.n_tiles)
    assert int(warp.n_tiles) == nt == sum(-(-int(c) // tile) for c in torch.bincount(flat, minlength=E))
    assert torch.equal(warp.counts, other.counts) and torch.equal(warp.offsets, other.offsets)
    assert torch.equal(warp.sorted_pairs[:P], other.sorted_pairs[:P]) and torch.equal(warp.pos_of_pair[:P], other.pos_of_pair[:P])
    for a, b in ((warp.tile_group, other.tile_group), (warp.tile_row0, other.tile_row0), (warp.tile_rows, other.tile_rows)):
        assert torch.equal(a[:nt], b[:nt])


def test_embed_records_a_bad_token_instead_of_faulting():
    o = ops()
    table = rnd(10, 32).to(DEV)
    res = torch.empty(2, 32, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.embed_rows(table, torch.tensor([3, 10], dtype=torch.int32, device=DEV), res, status)
    assert int(status) == 1


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    o = ops()
    gu = rnd(7, 2 * 150, seed=5).to(dtype)
    out = torch.empty(7, 150, dtype=dtype, device=DEV)
    o.silu_mul(gu.to(DEV), out)
    g, u = gu.float()[:, :150], gu.float()[:, 150:]
    close(out, torch.nn.functional.silu(g) * u, dtype)


def plain_activation(name, g):
    """The gate activations a gated feed-forward may name, in plain torch."""
    return {"silu": torch.nn.functional.silu, "gelu": lambda t: torch.nn.functional.gelu(t),
            "relu2": lambda t: torch.relu(t) ** 2, "identity": lambda t: t}[name](g)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["silu", "gelu", "relu2", "identity"])
def test_gate_activations(dtype, act):
    o = ops()
    gu = rnd(9, 2 * 150, seed=5, scale=1.5).to(dtype)
    out = torch.empty(9, 150, dtype=dtype, device=DEV)
    o.gated_mul(gu.to(DEV), out, o.activation_code(act))
    g, u = gu.float()[:, :150], gu.float()[:, 150:]
    close(out, plain_activation(act, g) * u, dtype, act)
    with pytest.raises(o.KernelError, match="gate activation"):
        o.activation_code("swish7")
    with pytest.raises(o.KernelError, match="gate activation"):
        o.gated_mul(gu.to(DEV), out, 9)


@pytest.mark.parametrize("E,k,use_bias,normalize", [(12, 4, True, True), (12, 4, False, False), (70, 3, True, False),
                                                     (300, 6, False, True)])
def test_router_with_softmax_scores(E, k, use_bias, normalize):
    """The other scoring function: scores are the softmax over all experts' logits (32-bit); the bias still only moves
    the choice, the weights are the chosen scores, renormalised or not, times the scale. Alone and inside the norm kernel."""
    o = ops()
    R, H = 37, 136
    res0, w = rnd(R, H, seed=1), 1 + rnd(H, seed=2, scale=0.2)
    gate, bias = rnd(E, H, seed=7, scale=0.3), rnd(E, seed=8, scale=0.02)
    n32 = P.rms_norm(res0, w, 1e-5)
    logits = n32 @ gate.T
    score = torch.softmax(logits, -1)
    choice = score + bias if use_bias else score
    want_ids = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :k]
    want_w = torch.gather(score, 1, want_ids)
    if normalize:
        want_w = want_w / (want_w.sum(-1, keepdim=True) + 1e-6)
    want_w = want_w * 1.5
    ids = torch.empty(R, k, dtype=torch.int32, device=DEV)
    wts = torch.empty(R, k, dtype=torch.float32, device=DEV)
    o.router_topk(logits.to(DEV), bias.to(DEV) if use_bias else None, k, normalize, 1e-6, 1.5, ids, wts, scoring="softmax")
    assert torch.equal(ids.cpu().long(), want_ids)
    close(wts, want_w, torch.float32, "softmax routing weights")
    route = {"weight": gate.to(DEV), "bias": bias.to(DEV) if use_bias else None, "k": k, "normalize": normalize,
             "scoring": "softmax", "floor": 1e-6, "scale": 1.5,
             "ids": torch.empty(R, k, dtype=torch.int32, device=DEV), "wts": torch.empty(R, k, dtype=torch.float32, device=DEV)}
    out = torch.empty(R, H, dtype=torch.float32, device=DEV)
    o.add_rmsnorm(res0.clone().to(DEV), None, w.to(DEV), 1e-5, out, None, None, route)
    assert torch.equal(route["ids"].cpu().long(), want_ids)
    close(route["wts"], want_w, torch.float32, "softmax routing weights from the norm kernel")
    with pytest.raises(o.KernelError, match="scoring"):
        o.router_topk(logits.to(DEV), None, k, normalize, 1e-6, 1.5, ids, wts, scoring="sparsemax")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["gelu", "relu2", "identity"])
def test_grouped_products_with_other_gate_activations(dtype, act):
    o = ops()
    R, E, k, H, I = 40, 5, 2, 64, 24
    x = rnd(R, H, seed=11).to(dtype)
    w13 = rnd(E, 2 * I, H, seed=14, scale=0.3).to(dtype)
    ids = torch.stack([torch.randperm(E, generator=torch.Generator().manual_seed(r))[:k] for r in range(R)]).int().to(DEV)
    plan = o.MoePlan(R * k, E, o.simt_tile_rows(), DEV).build(ids)
    got = torch.empty(R * k, I, dtype=dtype, device=DEV)
    o.gemm_simt_grouped(x.to(DEV), plan.sorted_pairs, k, w13.to(DEV), got, plan, o.activation_code(act))
    order = plan.sorted_pairs[:R * k].cpu().long()
    xf, wf = x.float(), w13.float()
    flat = ids.cpu().reshape(-1).long()
    want = torch.stack([plain_activation(act, xf[p // k] @ wf[flat[p], :I].T) * (xf[p // k] @ wf[flat[p], I:].T) for p in order])
    close(got, want, dtype, act)


# ------------------------------------------------------------------------------------------ products
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 130, 77), (3, 64, 64), (8, 257, 100), (9, 130, 77), (70, 96, 200), (200, 33, 17),
                                   (5, 40, 600), (8, 32, 2048), (300, 64, 130), (2048, 32, 256)])
def test_gemm_simt(dtype, M, N, K):
    o = ops()
    x, w, b = rnd(M, K, seed=6).to(dtype), rnd(N, K, seed=7).to(dtype), rnd(N, seed=8)
    want = x.float() @ w.float().T + b
    for out_dtype in {dtype, torch.float32}:
        out = torch.empty(M, N, dtype=out_dtype, device=DEV)
        o.gemm_simt(x.to(DEV), w.to(DEV), b.to(DEV), out)
        close(out, want, out_dtype if dtype == torch.float32 else torch.bfloat16, f"{M}x{N}x{K}")
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    o.gemm_simt(x.to(DEV), w.to(DEV), None, out)
    close(out, x.float() @ w.float().T, dtype, "no bias")


def test_gemm_row_does_not_depend_on_the_other_rows():
    """A row of a tiled call equals the same row in a smaller tiled call bit for bit (the k order is fixed)."""
    o = ops()
    x, w = rnd(100, 300, seed=9).to(DEV), rnd(50, 300, seed=10).to(DEV)
    big = o.gemm_simt(x, w, None, torch.empty(100, 50, device=DEV))
    small = o.gemm_simt(x[60:75].contiguous(), w, None, torch.empty(15, 50, device=DEV))
    assert torch.equal(big[60:75], small)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("R,E,k,H,I", [(5, 4, 2, 48, 40), (70, 6, 3, 96, 72), (300, 40, 4, 64, 24), (1, 8, 8, 32, 16)])
def test_router_plan_experts_and_combine(dtype, R, E, k, H, I):
    """The expert path end to end against a loop over experts, and its plan against a stable sort."""
    o = ops()
    x = rnd(R, H, seed=11)
    gate, bias = rnd(E, H, seed=12, scale=0.3), rnd(E, seed=13, scale=0.2)
    w13, w2 = rnd(E, 2 * I, H, seed=14, scale=0.2).to(dtype), rnd(E, H, I, seed=15, scale=0.2).to(dtype)
    xd = x.to(dtype)
    logits = x @ gate.T
    ids = torch.empty(R, k, dtype=torch.int32, device=DEV)
    wts = torch.empty(R, k, dtype=torch.float32, device=DEV)
    for normalize, scale, use_bias in ((True, 1.0, True), (False, 2.5, False)):
        o.router_topk(logits.to(DEV), bias.to(DEV) if use_bias else None, k, normalize, 1e-6, scale, ids, wts)
        cfg = dict(num_experts_per_tok=k, use_expert_bias=use_bias, norm_topk_prob=normalize, routed_scaling_factor=scale)
        want_ids, want_w = P.route(x, {"gate.weight": gate, "expert_bias": bias}, "", cfg)
        assert torch.equal(ids.cpu().long(), want_ids), "chosen experts and their order"
        close(wts, want_w, torch.float32, "routing weights")
    plan = o.MoePlan(R * k, E, o.simt_tile_rows(), DEV).build(ids)
    flat = ids.cpu().reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    assert torch.equal(plan.sorted_pairs[:R * k].cpu().long(), order)
    assert torch.equal(plan.counts.cpu().long(), torch.bincount(flat, minlength=E))
    assert torch.equal(plan.pos_of_pair[:R * k].cpu().long()[order], torch.arange(R * k))
    nt = int(plan.n_tiles)
    assert nt == sum(-(-int(c) // plan.tile_m) for c in plan.counts.cpu()) and nt <= plan.max_tiles
    covered = sum(int(r) for r in plan.tile_rows[:nt].cpu())
    assert covered == R * k
    act = torch.empty(R * k, I, dtype=dtype, device=DEV)
    o.gemm_simt_grouped(xd.to(DEV), plan.sorted_pairs, k, w13.to(DEV), act, plan, True)
    y = torch.empty(R * k, H, dtype=torch.float32, device=DEV)
    o.gemm_simt_grouped(act, None, 1, w2.to(DEV), y, plan, False)
    out = torch.empty(R, H, dtype=torch.float32, device=DEV)
    o.moe_combine(y, plan, ids, wts, out)
    want = torch.zeros(R, H)
    xf, w13f, w2f = xd.float(), w13.float(), w2.float()
    wc = wts.cpu()
    for e in range(E):
        rows, slot = torch.where(ids.cpu() == e)
        if rows.numel():
            h = torch.nn.functional.silu(xf[rows] @ w13f[e, :I].T) * (xf[rows] @ w13f[e, I:].T)
            if dtype == torch.bfloat16:
                h = h.to(dtype).float()
            want.index_add_(0, rows, (h @ w2f[e].T) * wc[rows, slot, None])
    close(out, want, dtype, "experts")


def test_router_ties_and_many_experts():
    o = ops()
    for E, k in ((8, 3), (130, 5), (1000, 32)):
        logits = torch.zeros(4, E)
        logits[1, E - 1] = 1.0
        ids = torch.empty(4, k, dtype=torch.int32, device=DEV)
        wts = torch.empty(4, k, dtype=torch.float32, device=DEV)
        o.router_topk(logits.to(DEV), None, k, True, 1e-6, 1.0, ids, wts)
        assert ids[0].tolist() == list(range(k)), "equal scores: the lower ids, in order"
        assert ids[1].tolist() == [E - 1] + list(range(k - 1))
    with pytest.raises(o.KernelError, match="experts"):
        o.router_topk(torch.zeros(1, 2000, device=DEV), None, 2, True, 1e-6, 1.0, ids, wts)


# ------------------------------------------------------------------------------------------ short conv
def plain_conv_with_state(bcx, taps_w, bias, state, K):
    """Rows of one request after `state` [K-1, H] (oldest first): (y [n, H], new state)."""
    H = bcx.shape[1] // 3
    bx = bcx[:, :H] * bcx[:, 2 * H:]
    full = torch.cat([state, bx], 0)
    y = torch.stack([(full[t:t + K] * taps_w.T).sum(0) for t in range(bx.shape[0])])
    if bias is not None:
        y = y + bias
    return bcx[:, H:2 * H] * y, full[-(K - 1):]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("K,H,use_bias", [(3, 200, False), (4, 96, True), (2, 64, False), (7, 300, True)])
def test_short_conv_mixed_batch_and_state(dtype, K, H, use_bias):
    """Three requests in one call: a new one with a portion shorter than the taps, one that continues from its
    slot with a single row, one that continues with a long portion. A stale slot must not leak into a new one."""
    o = ops()
    lens, starts = [2, 1, 19], [0, 5, 3]
    R = sum(lens)
    bcx = rnd(R, 3 * H, seed=20).to(dtype)
    taps_w, bias = rnd(H, K, seed=21), (rnd(H, seed=22) if use_bias else None)
    slots = [2, 0, 3]
    state = rnd(5, K - 1, H, seed=23)                 # slot 2 holds junk that a sequence starting at 0 must not read
    row_start = [0, 2, 3, R]
    req_of_row = sum(([b] * n for b, n in enumerate(lens)), [])
    positions = sum((list(range(s, s + n)) for s, n in zip(starts, lens)), [])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    st = state.clone().to(DEV)
    y = torch.empty(R, H, dtype=dtype, device=DEV)
    args = (bcx.to(DEV), taps_w.to(DEV), bias.to(DEV) if use_bias else None, st, i32(slots), i32(req_of_row),
            i32(row_start), i32(positions), y)
    o.short_conv(*args)
    o.short_conv_state(bcx.to(DEV), st, i32(slots), i32(row_start), i32(positions), 3, H, K)
    for b in range(3):
        old = state[slots[b]].clone()
        if starts[b] < K - 1:                          # inputs before position 0 are zero
            old[:K - 1 - starts[b]] = 0
        rows = slice(row_start[b], row_start[b + 1])
        want_y, want_state = plain_conv_with_state(bcx[rows].float(), taps_w, bias, old, K)
        close(y[rows], want_y, dtype, f"request {b}")
        close(st[slots[b]], want_state, torch.float32, f"state of request {b}")
    assert torch.equal(st[1].cpu(), state[1]) and torch.equal(st[4].cpu(), state[4]), "other slots are untouched"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("K,H,use_bias", [(3, 200, False), (4, 96, True), (2, 64, False), (7, 304, True), (3, 2048, False)])
def test_short_conv_of_long_portions_walks_runs_of_rows(dtype, K, H, use_bias):
    """Portions of many rows (the kernel form in which a thread walks eight consecutive rows with the last inputs in
    registers): requests whose edges fall inside a run, a new sequence shorter than the taps, one that starts at
    position 1, a single row between long portions, a last run that is not full; against the plain formula and, bit
    for bit, against the row-by-row kernel (the same rows given in two calls too short for the run form)."""
    o = ops()
    lens, starts, slots = [37, 2, 64, 1, 30, 11], [0, 0, 5, 9, 1, 3], [2, 0, 3, 5, 1, 6]
    R = sum(lens)
    bcx = rnd(R, 3 * H, seed=20).to(dtype)
    taps_w, bias = rnd(H, K, seed=21), (rnd(H, seed=22) if use_bias else None)
    state = rnd(7, K - 1, H, seed=23)
    row_start = [0]
    for n in lens:
        row_start.append(row_start[-1] + n)
    req_of_row = sum(([b] * n for b, n in enumerate(lens)), [])
    positions = sum((list(range(s0, s0 + n)) for s0, n in zip(starts, lens)), [])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    dev = lambda t: None if t is None else t.to(DEV)
    y = torch.full((R, H), float("nan"), dtype=dtype, device=DEV)
    o.short_conv(dev(bcx), dev(taps_w), dev(bias), dev(state), i32(slots), i32(req_of_row), i32(row_start), i32(positions), y)
    for b in range(len(lens)):
        old = state[slots[b]].clone()
        if starts[b] < K - 1:
            old[:K - 1 - starts[b]] = 0
        rows = slice(row_start[b], row_start[b + 1])
        want_y, _ = plain_conv_with_state(bcx[rows].float(), taps_w, bias, old, K)
        close(y[rows], want_y, dtype, f"request {b}")
    # the same numbers as the row-by-row kernel: every request alone in a call of few rows, its state advanced by hand
    for b in (1, 3, 5):
        rows = slice(row_start[b], row_start[b + 1])
        alone = torch.empty(lens[b], H, dtype=dtype, device=DEV)
        o.short_conv(dev(bcx[rows]), dev(taps_w), dev(bias), dev(state), i32([slots[b]]), i32([0] * lens[b]), i32([0, lens[b]]),
                     i32(positions[rows]), alone)
        assert torch.equal(alone, y[rows]), b


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("K,H,use_bias", [(3, 200, False), (4, 96, True), (2, 64, False), (7, 300, True)])
def test_short_conv_of_single_rows_in_one_kernel(dtype, K, H, use_bias):
    """A step of one row a request (decoding) runs one kernel for the convolution and the state's shift: the same
    numbers, bit for bit, as the two general kernels, from a stored projection and from its partial sums; sequences
    at their first positions (inputs before position 0 are zero whatever the slot holds) beside later ones."""
    o = ops()
    starts, slots = [0, 1, 2, 5, 40], [2, 0, 3, 4, 6]
    R = len(starts)
    parts = torch.stack([rnd(R, 3 * H, seed=24 + i) for i in range(3)])           # [3, R, 3H] partial sums
    total = torch.zeros(R, 3 * H)
    for part in parts:
        total += part
    bcx = total.to(dtype)
    taps_w, bias = rnd(H, K, seed=21), (rnd(H, seed=22) if use_bias else None)
    state = rnd(7, K - 1, H, seed=23)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    dev = lambda t: None if t is None else t.to(DEV)
    st_two, y_two = state.clone().to(DEV), torch.empty(R, H, dtype=dtype, device=DEV)
    o.short_conv(bcx.to(DEV), dev(taps_w), dev(bias), st_two, i32(slots), i32(list(range(R))), i32(list(range(R + 1))),
                 i32(starts), y_two)
    o.short_conv_state(bcx.to(DEV), st_two, i32(slots), i32(list(range(R + 1))), i32(starts), R, H, K)
    for source in ("stored", "partial sums"):
        given = bcx.to(DEV) if source == "stored" else o.PartialSums(parts.to(DEV).contiguous(), 3, R, 3 * H,
                                                                      None if dtype == torch.float32 else dtype)
        st, y = state.clone().to(DEV), torch.empty(R, H, dtype=dtype, device=DEV)
        o.short_conv_decode(given, dev(taps_w), dev(bias), st, i32(slots), i32(list(range(R))), i32(starts), y)
        assert torch.equal(y, y_two), source
        assert torch.equal(st, st_two), source
        kept = state.clone().to(DEV)
        o.short_conv_decode(given, dev(taps_w), dev(bias), kept, i32(slots), i32(list(range(R))), i32(starts), y,
                            write_state=False)
        assert torch.equal(y, y_two) and torch.equal(kept.cpu(), state), "a site that reads another's state leaves it"


# ------------------------------------------------------------------------------------------ attention
def plain_attention(q, k, v, scale, window=None):
    """q [T, Hq, D] for the last T positions of a sequence whose keys k, v [L, Hk, D] are all given."""
    T, Hq, D = q.shape
    L, Hk = k.shape[0], k.shape[1]
    ks, vs = k.repeat_interleave(Hq // Hk, 1), v.repeat_interleave(Hq // Hk, 1)
    s = torch.einsum("thd,shd->hts", q, ks) * scale
    qpos = torch.arange(L - T, L)[:, None]
    kpos = torch.arange(L)[None, :]
    hidden = kpos > qpos
    if window:
        hidden = hidden | (kpos <= qpos - window)
    s = s.masked_fill(hidden[None], float("-inf"))
    return torch.einsum("hts,shd->thd", torch.softmax(s, -1), vs)


def paged_setup(seqs, Hk, D, page, dtype, seed):
    """Random K/V for sequences of the given lengths scattered over shuffled pages: (k_cache, v_cache, table, ks, vs)."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-L // page) for L in seqs) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.zeros(n_pages, Hk, page, D)
    vc = torch.zeros(n_pages, Hk, page, D)
    width = max(-(-L // page) for L in seqs) + 1
    table = torch.full((len(seqs), width), -1, dtype=torch.int32)
    ks, vs = [], []
    for b, L in enumerate(seqs):
        k = (torch.randn(L, Hk, D, generator=g)).to(dtype).float()
        v = (torch.randn(L, Hk, D, generator=g)).to(dtype).float()
        for j in range(-(-L // page)):
            pg = perm.pop()
            table[b, j] = pg
            n = min(page, L - j * page)
            kc[pg, :, :n] = k[j * page:j * page + n].transpose(0, 1)
            vc[pg, :, :n] = v[j * page:j * page + n].transpose(0, 1)
        ks.append(k)
        vs.append(v)
    return kc.to(dtype), vc.to(dtype), table, ks, vs


KERNELS = ["simt", "split"]


def attend(o, kind, q, kc, vc, table, page, req_of_row, positions, scale, window, out, status):
    """The plain CUDA-core kernel or the split (flash-decoding) kernel, the latter with scratch sized for the call."""
    if kind == "simt":
        return o.paged_attention_simt(q, kc, vc, table, page, req_of_row, positions, scale, window, out, status)
    spans = o.attention_spans(int(positions.max()) + 1)
    R, Hq, D = q.shape
    scratch = torch.full((o.attention_scratch_floats(R, Hq, D, spans),), float("nan"), device=DEV)
    return o.paged_attention_split(q, kc, vc, table, page, req_of_row, positions, scale, window, out, scratch, spans, status)


@pytest.mark.parametrize("kind", KERNELS)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hk,D,page,window", [(6, 2, 48, 16, None), (5, 5, 16, 16, None), (8, 1, 128, 32, None),
                                                 (4, 2, 64, 16, 37), (3, 1, 256, 64, None), (4, 4, 80, 16, 16),
                                                 (24, 2, 32, 16, None)])
def test_paged_attention_mixed_rows(kind, dtype, Hq, Hk, D, page, window):
    """A decode row at a long context, a prompt portion in the middle of a sequence, and a sequence's first rows,
    in one call, against whole-sequence attention."""
    o = ops()
    seqs, news = [333, 90, 7], [1, 23, 7]              # context after the step, rows in the step
    kc, vc, table, ks, vs = paged_setup(seqs, Hk, D, page, dtype, seed=30)
    R = sum(news)
    q = rnd(R, Hq, D, seed=31).to(dtype)
    req_of_row = sum(([b] * n for b, n in enumerate(news)), [])
    positions = sum((list(range(L - n, L)) for L, n in zip(seqs, news)), [])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    out = torch.empty(R, Hq, D, dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 0.7 / math.sqrt(D)
    attend(o, kind, q.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), page, i32(req_of_row), i32(positions), scale,
           window, out, status)
    assert int(status) == 0
    at = 0
    for b, (L, n) in enumerate(zip(seqs, news)):
        want = plain_attention(q[at:at + n].float(), ks[b], vs[b], scale, window)
        close(out[at:at + n], want, dtype, f"sequence {b}")
        at += n


@pytest.mark.parametrize("kind", KERNELS)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 15, 16, 17, 255, 256, 300, 511])
def test_one_far_key_stands_out(kind, dtype, far):
    """Among 512 keys, one key is made to match the query so strongly that the output must be its value: a key
    skipped or read from the wrong page (a page's edge, a chunk's edge) shows at once."""
    o = ops()
    Hq, Hk, D, page, L = 4, 2, 64, 16, 512
    kc, vc, table, ks, vs = paged_setup([L], Hk, D, page, dtype, seed=40 + far)
    q = rnd(1, Hq, D, seed=41).to(dtype).float()
    # make key `far` of both KV heads equal to 4 x the queries' mean direction
    direction = q.mean(1)[0]
    pg, off = int(table[0, far // page]), far % page
    kc[pg, :, off] = (4 * direction).to(dtype)
    ks[0][far] = (4 * direction).to(dtype).float()
    out = torch.empty(1, Hq, D, dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    attend(o, kind, q.to(dtype).to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), page, i32([0]), i32([L - 1]), 1.0, None,
           out, status)
    want = plain_attention(q, ks[0], vs[0], 1.0)
    close(out, want, dtype, f"far key {far}")
    weight = torch.softmax(torch.einsum("hd,shd->hs", q[0], ks[0].repeat_interleave(2, 1)), -1)[:, far]
    assert float(weight.min()) > 0.5, "the test's key does dominate"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 700, 256, 257])
def test_split_kernel_over_many_spans(dtype, window):
    """Contexts of several 256-key spans, with and without a window whose edge falls inside a span, and rows of
    one call that need different numbers of spans."""
    o = ops()
    Hq, Hk, D, page = 8, 2, 64, 16
    seqs, news = [1500, 300, 1024], [2, 1, 3]
    kc, vc, table, ks, vs = paged_setup(seqs, Hk, D, page, dtype, seed=45)
    R = sum(news)
    q = rnd(R, Hq, D, seed=46).to(dtype)
    req_of_row = sum(([b] * n for b, n in enumerate(news)), [])
    positions = sum((list(range(L - n, L)) for L, n in zip(seqs, news)), [])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    out = torch.full((R, Hq, D), float("nan"), dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    attend(o, "split", q.to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), page, i32(req_of_row), i32(positions), 0.125,
           window, out, status)
    assert int(status) == 0
    at = 0
    for b, (L, n) in enumerate(zip(seqs, news)):
        close(out[at:at + n], plain_attention(q[at:at + n].float(), ks[b], vs[b], 0.125, window), dtype, f"sequence {b}")
        at += n


@pytest.mark.parametrize("kind", KERNELS)
@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edge(kind, dtype):
    """With a window of w the key w positions back is out and the one w-1 back is in; pages wholly behind the
    window may be gone (-1 in the table)."""
    o = ops()
    Hq, Hk, D, page, L, w = 2, 1, 32, 16, 100, 20
    kc, vc, table, ks, vs = paged_setup([L], Hk, D, page, dtype, seed=50)
    q = rnd(1, Hq, D, seed=51).to(dtype).float()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for hot in (L - w, L - w - 1):                      # first position inside the window, last one outside
        k2 = [ks[0].clone()]
        k2[0][hot] = (6 * q.mean(1)[0]).to(dtype).float()
        kc2 = kc.clone()
        kc2[int(table[0, hot // page]), :, hot % page] = k2[0][hot].to(dtype)
        t2 = table.clone()
        t2[0, :(L - w) // page] = -1                     # pages the window has passed
        out = torch.empty(1, Hq, D, dtype=dtype, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        attend(o, kind, q.to(dtype).to(DEV), kc2.to(DEV), vc.to(DEV), t2.to(DEV), page, i32([0]), i32([L - 1]), 1.0, w,
               out, status)
        assert int(status) == 0
        close(out, plain_attention(q, k2[0], vs[0], 1.0, w), dtype, f"hot key at {hot}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hk,D,rot", [(6, 2, 48, 48), (3, 1, 32, 16), (4, 4, 128, 128)])
def test_qk_prepare_norm_rotary_and_page_write(dtype, Hq, Hk, D, rot):
    o = ops()
    page, seqs, news = 16, [40, 17], [9, 17]
    R = sum(news)
    qkv = rnd(R, (Hq + 2 * Hk) * D, seed=60).to(dtype)
    qw, kw = 1 + rnd(D, seed=61, scale=0.2), 1 + rnd(D, seed=62, scale=0.2)
    theta, eps = 5e4, 2e-5
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    table = torch.tensor([[4, 1, 6, -1], [0, 5, -1, -1]], dtype=torch.int32)
    req_of_row = sum(([b] * n for b, n in enumerate(news)), [])
    positions = sum((list(range(L - n, L)) for L, n in zip(seqs, news)), [])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    kc = torch.zeros(8, Hk, page, D, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(R, Hq, D, dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.qk_prepare(qkv.to(DEV), qw.to(DEV), kw.to(DEV), eps, inv_freq.to(DEV), rot, i32(positions), i32(req_of_row),
                 table.to(DEV), page, q_out, kc, vc, None, None, Hq, Hk, D, status)
    assert int(status) == 0
    x = qkv.float()
    q = P.rms_norm(x[:, :Hq * D].view(R, Hq, D), qw, eps)
    k = P.rms_norm(x[:, Hq * D:(Hq + Hk) * D].view(R, Hk, D), kw, eps)
    v = x[:, (Hq + Hk) * D:].view(R, Hk, D)
    pos = torch.tensor(positions)
    f = pos.float()[:, None] * inv_freq[None, :]
    cos, sin = torch.cat([f, f], -1).cos()[:, None, :], torch.cat([f, f], -1).sin()[:, None, :]

    def rope(t):
        a, rest = t[..., :rot], t[..., rot:]
        return torch.cat([a * cos + P.rotate_half(a) * sin, rest], -1)
    close(q_out, rope(q), dtype, "q")
    kk, vv = rope(k), v
    for r in range(R):
        b, p = req_of_row[r], positions[r]
        pg = int(table[b, p // page])
        close(kc[pg, :, p % page], kk[r], dtype, f"k row {r}")
        close(vc[pg, :, p % page], vv[r], dtype, f"v row {r}")
    # the unfused pair: plain outputs, then the page write
    k_out = torch.empty(R, Hk, D, dtype=dtype, device=DEV)
    v_out = torch.empty(R, Hk, D, dtype=dtype, device=DEV)
    o.qk_prepare(qkv.to(DEV), qw.to(DEV), kw.to(DEV), eps, None, 0, i32(positions), i32(req_of_row), None, 0, q_out,
                 None, None, k_out, v_out, Hq, Hk, D, status)
    close(k_out, k, dtype, "k without rotation")
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    o.kv_store(k_out, v_out, i32(positions), i32(req_of_row), table.to(DEV), page, kc2, vc2, status)
    r = R - 1
    pg = int(table[1, positions[r] // page])
    assert torch.equal(kc2[pg, :, positions[r] % page], k_out[r]) and int(status) == 0
    # a write to a position without a page is recorded, not performed
    o.kv_store(k_out[:1], v_out[:1], i32([50]), i32([1]), table.to(DEV), page, kc2, vc2, status)
    assert int(status) == 2
    # so are a table entry that names no page of the pool and a position past the table's width (a corrupted table
    # or position must end as a status word, never as a wild address)
    before = (kc2.clone(), vc2.clone())
    wild = table.clone()
    wild[1, positions[r] // page] = kc2.shape[0] + 1000
    for tab, pos in ((wild, positions[r]), (table, table.shape[1] * page + 5)):
        status.zero_()
        o.kv_store(k_out[:1], v_out[:1], i32([pos]), i32([1]), tab.to(DEV), page, kc2, vc2, status)
        assert int(status) == 2
        status.zero_()
        o.qk_prepare(qkv[:1].to(DEV), qw.to(DEV), kw.to(DEV), eps, inv_freq.to(DEV), rot, i32([pos]), i32([1]), tab.to(DEV),
                     page, q_out[:1], kc2, vc2, None, None, Hq, Hk, D, status)
        assert int(status) == 2
        out1 = torch.zeros(1, Hq, D, dtype=dtype, device=DEV)
        for kind in KERNELS:
            status.zero_()
            attend(o, kind, q_out[:1], kc2, vc2, tab.to(DEV), page, i32([1]), i32([pos]), 1.0, None, out1, status)
            assert int(status) == 3, kind
    assert torch.equal(kc2, before[0]) and torch.equal(vc2, before[1])


def test_refused_sizes_are_clear_errors():
    o = ops()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = torch.zeros(1, 2, 24, device=DEV)
    kc = torch.zeros(2, 2, 16, 24, device=DEV)
    with pytest.raises(o.KernelError, match="head size 24"):
        o.paged_attention_simt(q, kc, kc, i32([[0]]), 16, i32([0]), i32([0]), 1.0, None, torch.empty_like(q), status)
    with pytest.raises(o.KernelError, match="taps"):
        o.short_conv(torch.zeros(1, 96, device=DEV), torch.zeros(32, 17, device=DEV), None, torch.zeros(1, 16, 32, device=DEV),
                     i32([0]), i32([0]), i32([0, 1]), i32([0]), torch.empty(1, 32, device=DEV))
    with pytest.raises(o.KernelError, match="CUDA"):
        o.gemm_simt(torch.zeros(1, 4), torch.zeros(2, 4), None, torch.zeros(1, 2))


# ------------------------------------------------------------------------------------------ sampling
def test_argmax_and_sampling_match_the_plain_draws():
    o = ops()
    V, n = 5003, 12
    logits = rnd(n, V, seed=70, scale=2.5)
    logits[3, 77] = logits[3, 4000] = logits[3].max() + 1     # a tie: the lower index
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    o.argmax(logits.to(DEV), out)
    assert out.tolist() == [77 if i == 3 else int(logits[i].argmax()) for i in range(n)]
    wide = rnd(3, 40000, seed=71)                              # a width that 16-byte loads take
    wide[1, 39999] = wide[1, 5] = wide[1].max() + 1
    wide[2, 7] = float("nan")
    o.argmax(wide.to(DEV), out[:3])
    assert out[:3].tolist() == [int(wide[0].argmax()), 5, int(torch.nan_to_num(wide[2], nan=-1e30).argmax())]
    temps = [0.0, 0.7, 1.0, 1.3, 0.7, 0.7, 1.0, 0.5, 2.0, 1.0, 0.9, 0.0]
    top_k = [0, 0, 50, 0, 5, 0, 20, 1, 0, 0, 3, 7]
    top_p = [1.0, 1.0, 1.0, 0.9, 1.0, 0.5, 0.95, 1.0, 0.3, 1.0, 0.8, 0.2]
    min_p = [0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.1, 0.05, 0.0]
    seeds = [11 * i + 3 for i in range(n)]
    pos = [5 * i for i in range(n)]
    f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
    o.sample(logits.to(DEV), f32(temps), torch.tensor(top_k, dtype=torch.int32, device=DEV), f32(top_p), f32(min_p),
             torch.tensor(seeds, dtype=torch.int64, device=DEV), torch.tensor(pos, dtype=torch.int32, device=DEV), out)
    got = out.tolist()
    for i in range(n):
        want = P.sample(logits[i], temps[i], top_k[i], top_p[i], min_p[i], seeds[i], pos[i])
        if got[i] != want:
            # the only allowed difference: a token at a filter's edge, kept by one side and not the other
            keep = P.kept_tokens(logits[i], temps[i], top_k[i], top_p[i], min_p[i])
            assert temps[i] > 0 and bool(keep[got[i]]) , (i, got[i], want)
    assert sum(g == P.sample(logits[i], temps[i], top_k[i], top_p[i], min_p[i], seeds[i], pos[i])
               for i, g in enumerate(got)) >= n - 1


def test_sampling_follows_the_distribution_and_the_filters():
    o = ops()
    V, n = 50, 20000
    row = torch.tensor([math.log(i + 1.0) for i in range(V)])
    logits = row.repeat(n, 1).to(DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ones = torch.ones(n, device=DEV)
    i32z = torch.zeros(n, dtype=torch.int32, device=DEV)
    seeds = torch.arange(n, dtype=torch.int64, device=DEV) * 7919 + 1
    o.sample(logits, ones, i32z, ones, ones * 0, seeds, i32z, out)
    freq = torch.bincount(out.cpu().long(), minlength=V).float() / n
    p = torch.softmax(row, -1)
    assert float((freq - p).abs().max()) < 0.01
    o.sample(logits, ones, i32z + 5, ones, ones * 0, seeds, i32z, out)
    assert set(out.tolist()) <= set(range(V - 5, V))
    o.sample(logits, ones, i32z, ones * 0.5, ones * 0, seeds, i32z, out)
    kept = P.kept_tokens(row, 1.0, 0, 0.5, 0.0)
    assert set(out.tolist()) <= set(torch.nonzero(kept).reshape(-1).tolist())
    # same seed and position: the same token whatever else is in the batch; another position: other noise
    a = out.clone()
    o.sample(logits[:7], ones[:7], i32z[:7], ones[:7] * 0.5, ones[:7] * 0, seeds[:7], i32z[:7], out[:7])
    assert torch.equal(a[:7], out[:7])
    o.sample(logits, ones, i32z, ones, ones * 0, seeds, i32z + 1, out)
    assert not torch.equal(a, out)
