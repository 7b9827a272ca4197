"""A plain, slow implementation of the LFM2 MoE forward pass: whole sequences, no cache, one function per
part, plain torch on the CPU. It shares no code with the package: tests compare the engine with it.

Every function is written from the reference's formulas and cites where (paths are the reference
project's own). The reference's model code imports on the CPU here, and this file was compared with it
once on a tiny random model: `tests/golden/make_golden.py` ran `Lfm2MoeRef` (engine/models/lfm2_moe/ref.py)
and stored its logits in `tests/golden/tiny_a_reference.npz`; `tests/test_plain.py` holds this file to
those numbers. Three options the reference refuses for this family (engine/models/lfm2_moe/config.py:47-48:
conv bias, un-normalised top-k weights, an untied head) cannot be run through that class; they rest on the
formulas, read where the reference's sibling families implement the same options: a causal depthwise
convolution's bias is added to the tap sum before what follows it (engine/models/nemotron_h/ref.py:195-201),
projection biases are those of a linear layer, un-normalised top-k weights skip the division and nothing else
(engine/models/flashnext/ref.py:484-485; the scaling is a line of its own, engine/models/lfm2_moe/ref.py:197),
and the head reads `lm_head.weight` when there is one (engine/models/lfm2_moe/ref.py:96-97).

Weights are a dict of canonical names (the checkpoint's without `model.`), as in ref.py:21-29.
The configuration is a plain dict with config.json's keys.
"""

from __future__ import annotations

import math

import torch


def cfg_get(cfg: dict, key: str, default=None):
    return cfg[key] if key in cfg and cfg[key] is not None else default


def rope_theta(cfg: dict) -> float:
    # engine/models/lfm2_moe/config.py:155: rope_parameters.rope_theta, else rope_theta, else 1e6
    rope = cfg.get("rope_parameters") or {}
    return float(rope.get("rope_theta", cfg.get("rope_theta", 1e6)))


def layer_kinds(cfg: dict) -> list[str]:
    # engine/models/lfm2_moe/config.py:129-133
    if cfg.get("layer_types") is not None:
        return list(cfg["layer_types"])
    idx = set(cfg.get("full_attn_idxs") or [])
    return ["full_attention" if i in idx else "conv" for i in range(cfg["num_hidden_layers"])]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """engine/models/lfm2_moe/ref.py:105-109: mean of squares and rsqrt in 32-bit, cast back, times plain w."""
    dt = x.dtype
    h = x.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return w * h.to(dt)


def rotary_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """engine/models/lfm2_moe/ref.py:84 and :111-116: inv_freq_i = theta^(-2i/D); the two halves share a frequency."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    f = positions.float()[:, None] * inv_freq[None, :]
    emb = torch.cat([f, f], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """engine/models/lfm2_moe/ref.py:118-120."""
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def short_conv(n: torch.Tensor, W: dict, p: str, taps: int, bias: bool) -> torch.Tensor:
    """The double-gated short conv of a whole sequence [T, H] from a zero state
    (engine/models/lfm2_moe/ref.py:134-151): bcx = in_proj(n); B, C, x = thirds; bx = B * x; the window of row t
    is the last `taps` inputs ending at t (zeros before the sequence), tap taps-1 multiplies the row itself;
    y = C * conv; out = out_proj(y). With `bias` (not in the reference): the in_proj, conv and out_proj biases."""
    T, H = n.shape
    bcx = n @ W[p + "in_proj.weight"].T
    if bias:
        bcx = bcx + W[p + "in_proj.bias"]
    B, C, x = bcx[:, :H], bcx[:, H:2 * H], bcx[:, 2 * H:]
    bx = B * x
    wc = W[p + "conv.weight"].reshape(H, taps)
    padded = torch.cat([torch.zeros(taps - 1, H, dtype=bx.dtype), bx], 0)
    out = torch.zeros(T, H, dtype=bx.dtype)
    for t in range(T):
        win = padded[t:t + taps]                     # [taps, H], oldest first
        out[t] = (win * wc.T).sum(0)
    if bias:
        out = out + W[p + "conv.bias"]
    y = C * out
    y = y @ W[p + "out_proj.weight"].T
    if bias:
        y = y + W[p + "out_proj.bias"]
    return y


def attention(n: torch.Tensor, W: dict, p: str, cfg: dict, window: int | None = None) -> torch.Tensor:
    """Causal grouped-query attention of a whole sequence [T, H] (engine/models/lfm2_moe/ref.py:153-178):
    per-head RMS norm of q and k, rotary on q and k, scores * D^-0.5, softmax in 32-bit, query head h reads
    KV head h // (Hq / Hk)."""
    T = n.shape[0]
    Hq, Hk = cfg["num_attention_heads"], cfg_get(cfg, "num_key_value_heads", cfg["num_attention_heads"])
    D = cfg_get(cfg, "head_dim", cfg["hidden_size"] // Hq)
    eps = cfg_get(cfg, "norm_eps", 1e-5)
    q = rms_norm((n @ W[p + "q_proj.weight"].T).view(T, Hq, D), W[p + "q_layernorm.weight"], eps)
    k = rms_norm((n @ W[p + "k_proj.weight"].T).view(T, Hk, D), W[p + "k_layernorm.weight"], eps)
    v = (n @ W[p + "v_proj.weight"].T).view(T, Hk, D)
    cos, sin = rotary_tables(torch.arange(T), D, rope_theta(cfg), n.dtype)
    cos, sin = cos[:, None, :], sin[:, None, :]
    q = q * cos + rotate_half(q) * sin
    k = k * cos + rotate_half(k) * sin
    g = Hq // Hk
    ks = k.repeat_interleave(g, dim=1)               # [T, Hq, D]
    vs = v.repeat_interleave(g, dim=1)
    s = torch.einsum("thd,shd->hts", q, ks) * (D ** -0.5)
    i = torch.arange(T)
    hidden = i[None, :] > i[:, None]                  # key after the query
    if window is not None:
        hidden = hidden | (i[None, :] <= i[:, None] - window)
    s = s.masked_fill(hidden[None], float("-inf"))
    a = torch.softmax(s, dim=-1, dtype=torch.float32).to(n.dtype)
    o = torch.einsum("hts,shd->thd", a, vs).reshape(T, Hq * D)
    return o @ W[p + "out_proj.weight"].T


def dense_mlp(n: torch.Tensor, W: dict, p: str) -> torch.Tensor:
    """engine/models/lfm2_moe/ref.py:180-183: w2(silu(w1 n) * (w3 n))."""
    return (torch.nn.functional.silu(n @ W[p + "w1.weight"].T) * (n @ W[p + "w3.weight"].T)) @ W[p + "w2.weight"].T


def route(n: torch.Tensor, W: dict, p: str, cfg: dict, forced: torch.Tensor | None = None
          ) -> tuple[torch.Tensor, torch.Tensor]:
    """(ids [T, k], weights [T, k]) (engine/models/lfm2_moe/ref.py:185-197): sigmoid scores; with an expert bias the
    choice is the top-k of score + bias and the weights are the chosen scores; weights / (sum + 1e-6) when
    normalised (always, in the reference); times routed_scaling_factor. Ties go to the lower expert id
    (engine/models/lfm2_moe/kernels.py:277). `forced` [T, k] replaces the choice (the weights are still this
    function's own): what another implementation chose at a near tie."""
    k = cfg_get(cfg, "num_experts_per_tok", 4)
    logits = n @ W[p + "gate.weight"].T
    s = logits.sigmoid()
    choice = s + W[p + "expert_bias"] if cfg_get(cfg, "use_expert_bias", True) else s
    # stable descending sort: the lower id first among equals
    ids = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :k]
    if forced is not None:
        ids = forced.long()
    w = torch.gather(s, 1, ids)
    if cfg_get(cfg, "norm_topk_prob", True):
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-6)
    return ids, w * float(cfg_get(cfg, "routed_scaling_factor", 1.0))


def expert_mlp(x: torch.Tensor, W: dict, p: str, e: int) -> torch.Tensor:
    """engine/models/lfm2_moe/ref.py:199-205."""
    q = f"{p}experts.{e}."
    return (torch.nn.functional.silu(x @ W[q + "w1.weight"].T) * (x @ W[q + "w3.weight"].T)) @ W[q + "w2.weight"].T


def routing_margin(n: torch.Tensor, W: dict, p: str, cfg: dict) -> torch.Tensor:
    """Per row, the gap between the k-th and the (k+1)-th choice score: how far the row is from another choice
    of experts (0 when every expert is chosen anyway)."""
    k = cfg_get(cfg, "num_experts_per_tok", 4)
    s = (n @ W[p + "gate.weight"].T).sigmoid()
    choice = s + W[p + "expert_bias"] if cfg_get(cfg, "use_expert_bias", True) else s
    if k >= choice.shape[-1]:
        return torch.full((n.shape[0],), float("inf"))
    top = torch.sort(choice, dim=-1, descending=True).values
    return top[:, k - 1] - top[:, k]


def moe(n: torch.Tensor, W: dict, p: str, cfg: dict, margins: list | None = None,
        forced: torch.Tensor | None = None) -> torch.Tensor:
    """engine/models/lfm2_moe/ref.py:207-214: each chosen expert's output times its weight, added in ascending
    expert id. `margins`, when given, collects each layer's routing margins."""
    if margins is not None:
        margins.append(routing_margin(n, W, p, cfg))
    ids, w = route(n, W, p, cfg, forced)
    out = torch.zeros_like(n)
    for e in sorted(set(ids.reshape(-1).tolist())):
        rows, slot = torch.where(ids == e)
        out.index_add_(0, rows, expert_mlp(n[rows], W, p, e) * w[rows, slot, None])
    return out


def forward(cfg: dict, W: dict, tokens: list[int] | torch.Tensor, dtype=torch.float32,
            margins: list | None = None, forced_routes: dict | None = None, rows: list[int] | None = None) -> torch.Tensor:
    """Logits [T, vocab] (32-bit) of a whole sequence (engine/models/lfm2_moe/ref.py:218-241): embed; per layer
    n = norm(h), h += mixer(n), n = norm(h), h += ffn(n); final norm `embedding_norm`; head = lm_head.weight
    if the model has an untied head, else the embedding. `margins` collects the routing margins [T] of every
    MoE layer. `forced_routes` {layer index: ids [T, k]} replaces those layers' choice of experts. `rows`: the
    logits of these positions only (the head of a large vocabulary over thousands of rows is most of the work)."""
    W = {k: (v.to(dtype) if v.is_floating_point() and not k.endswith("expert_bias") else v) for k, v in W.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg_get(cfg, "norm_eps", 1e-5)
    kinds = layer_kinds(cfg)
    dense_layers = cfg_get(cfg, "num_dense_layers", 2)
    h = W["embed_tokens.weight"][tokens].to(dtype)
    for li, kind in enumerate(kinds):
        p = f"layers.{li}."
        n = rms_norm(h, W[p + "operator_norm.weight"], eps)
        if kind == "full_attention":
            h = h + attention(n, W, p + "self_attn.", cfg)
        else:
            h = h + short_conv(n, W, p + "conv.", cfg_get(cfg, "conv_L_cache", 3), bool(cfg.get("conv_bias", False)))
        n = rms_norm(h, W[p + "ffn_norm.weight"], eps)
        f = p + "feed_forward."
        forced = forced_routes.get(li) if forced_routes else None
        h = h + (moe(n, W, f, cfg, margins, forced) if li >= dense_layers else dense_mlp(n, W, f))
    if rows is not None:
        h = h[torch.as_tensor(rows, dtype=torch.long)]
    h = rms_norm(h, W["embedding_norm.weight"], eps)
    tied = cfg.get("tie_word_embeddings", cfg.get("tie_embedding", True))
    head = W["embed_tokens.weight"] if tied else W["lm_head.weight"]
    return (h @ head.T).float()


def greedy(cfg: dict, W: dict, prompt: list[int], steps: int, dtype=torch.float32) -> list[int]:
    """engine/spec.py:150-199 without the cache: the whole sequence is run again for every token."""
    seq, out = list(prompt), []
    for _ in range(steps):
        tok = int(forward(cfg, W, seq, dtype)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out


# ---- sampling (engine/sample.py:172-199, :311-322), with the engine's keyed noise restated ----
_M64 = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def keyed_uniform(seed: int, position: int, token: int) -> float:
    """Uniform in (0, 1) with 23 bits for (seed, position, token): the generator the sampling kernel documents."""
    key = _splitmix64((seed * 0x9E3779B97F4A7C15 + position + 1) & _M64)
    r = _splitmix64(key ^ (((token + 1) * 0xD1342543DE82EF95) & _M64))
    return ((r >> 41) + 0.5) / 8388608.0


def kept_tokens(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float) -> torch.Tensor:
    """Boolean mask of the tokens a draw may return (engine/sample.py:172-199): temperature, then min_p, then
    top-k, then top-p over the sorted remainder (keep a token while the mass before it does not exceed top_p)."""
    z = logits.double() / temperature
    keep = torch.ones_like(z, dtype=torch.bool)
    if min_p > 0:
        keep &= z >= z.max() + math.log(min_p)
    if top_k > 0:
        zz = z.masked_fill(~keep, float("-inf"))
        kth = torch.topk(zz, min(top_k, z.numel())).values[-1]
        keep &= zz >= kth
    if top_p < 1.0:
        zz = z.masked_fill(~keep, float("-inf"))
        sz, order = torch.sort(zz, descending=True)
        probs = torch.softmax(sz, dim=-1)
        before = torch.cumsum(probs, dim=-1) - probs
        kept_sorted = before <= top_p
        kept_sorted[0] = True
        mask = torch.zeros_like(keep)
        mask[order[kept_sorted]] = True
        keep &= mask
    return keep


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float, seed: int,
           position: int) -> int:
    """argmax of z + Gumbel noise over the kept tokens (engine/sample.py:311-322 with this engine's noise)."""
    if temperature <= 0:
        return int(logits.argmax())
    keep = kept_tokens(logits, temperature, top_k, top_p, min_p)
    z = logits.float() / temperature
    best, best_v = 0, -math.inf
    for i in torch.nonzero(keep).reshape(-1).tolist():
        u = keyed_uniform(seed, position, i)
        v = float(z[i]) - math.log(-math.log(u))
        if v > best_v:
            best, best_v = i, v
    return best


def penalize(logits: torch.Tensor, history: list[int], repetition: float = 1.0, presence: float = 0.0,
             frequency: float = 0.0, bias: dict | None = None) -> torch.Tensor:
    """A row of logits after `logit_bias` and the three penalties, given the tokens before it (prompt and generated):
    the bias is added first (engine/penalty.py:189-204, :291); then a token that the history holds has its logit
    multiplied by the repetition penalty if negative and divided by it otherwise, loses the presence penalty once,
    and the frequency penalty times its count (penalty.py:320-331; the counts are seeded from the prompt and grow
    with every committed token, penalty.py:206-232)."""
    out = logits.clone().float()
    for t, v in sorted((bias or {}).items()):
        out[t] += v
    counts = torch.zeros(out.numel(), dtype=torch.int64)
    for t in history:
        counts[t] += 1
    seen = counts > 0
    if repetition != 1.0:
        out = torch.where(seen, torch.where(out < 0, out * repetition, out / repetition), out)
    if presence != 0.0:
        out = out - presence * seen
    if frequency != 0.0:
        out = out - frequency * counts.float() * seen
    return out


def no_repeat_blocked(calls: list[list[int]], n: int, window: int = 2048) -> set[int]:
    """The tokens the no-repeat-n-gram rule penalises for the next draw, after the text was taken in by the `calls` one
    after the other (the prompt, then every committed token): the text is kept over a window (when it grows past
    `window` tokens at the end of a call, all but the last window // 2 are forgotten; engine/penalty.py:222-244), and a
    token is blocked when it followed the text's last n - 1 tokens somewhere in what is kept (penalty.py:246-276).
    Brute force over the kept text, no index."""
    kept: list[int] = []
    for ids in calls:
        kept.extend(ids)
        if len(kept) > window:
            del kept[:len(kept) - window // 2]
    L = n - 1
    if len(kept) < L:
        return set()
    tail = kept[-L:]
    return {kept[j + L] for j in range(len(kept) - L) if kept[j:j + L] == tail}


def pattern_ends(tokens: list[int], min_size: int, max_size: int, count: int) -> bool:
    """Whether the generated tokens end in one block of min_size..max_size tokens written `count` times over
    (engine/penalty.py:133-156)."""
    for size in range(min_size, max_size + 1):
        if len(tokens) >= size * count and tokens[-size * count:] == tokens[-size:] * count:
            return True
    return False
