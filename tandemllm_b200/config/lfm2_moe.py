"""The LFM2 / LFM2.5 MoE configuration (`model_type: lfm2_moe`, `Lfm2MoeForCausalLM`), typed.

Every size and constant the model uses is read here from the architecture's own config.json keys
and nowhere else; `to_spec()` turns it into the architecture-neutral `ModelSpec` the engine builds
from. Keys, defaults and checks follow the reference's reader (engine/models/lfm2_moe/config.py:33-48
KNOWN / IGNORED / FIXED, :126-169 `config_from_dict`, :172-193 `validate`): a key this reader does
not know stops the load with its name, and keys whose value would change the arithmetic are checked
against the values implemented.

Three options the reference pins to one value are implemented here with both values
(engine/models/lfm2_moe/config.py:47-48 refuses the other one):

  conv_bias            True: `conv.in_proj.bias [3H]`, `conv.conv.bias [H]` (added to the tap sum
                       before the C gate) and `conv.out_proj.bias [H]` are bound by name
  norm_topk_prob       False: the chosen router scores are not renormalised (still scaled by
                       `routed_scaling_factor`)
  tie_word_embeddings  False: `lm_head.weight [V, H]` must be present
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field

from .spec import LayerSpec, ModelSpec, PartSpec, plain_schedule

MODEL_TYPES = ("lfm2_moe",)
ARCHITECTURES = ("Lfm2MoeForCausalLM",)

KNOWN = {
    "hidden_size", "intermediate_size", "moe_intermediate_size", "num_hidden_layers", "num_attention_heads",
    "num_key_value_heads", "head_dim", "vocab_size", "norm_eps", "rope_parameters", "rope_theta",
    "max_position_embeddings", "layer_types", "full_attn_idxs", "conv_L_cache", "num_dense_layers", "num_experts",
    "num_experts_per_tok", "routed_scaling_factor", "use_expert_bias", "eos_token_id", "bos_token_id",
    "pad_token_id", "model_type", "architectures", "conv_bias", "norm_topk_prob", "tie_word_embeddings",
    "tie_embedding",
}
# training, other runtimes, or what tokenizer files own: read by nothing here
IGNORED = {
    "dtype", "torch_dtype", "initializer_range", "output_router_logits", "use_cache", "transformers_version",
    "block_dim", "block_ff_dim", "block_multiple_of", "block_ffn_dim_multiplier", "block_auto_adjust_ff_dim",
    "router_aux_loss_coef", "attention_dropout", "_name_or_path", "name_or_path",
}
# the one value implemented for keys that would change the arithmetic
FIXED = {"hidden_act": "silu", "attention_bias": False}

LAYER_KINDS = ("conv", "full_attention")


@dataclass
class Lfm2MoeConfig:
    hidden_size: int
    intermediate_size: int              # a dense layer's feed-forward width
    moe_intermediate_size: int          # one expert's width
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    layer_types: list[str]              # "conv" | "full_attention", one per layer
    norm_eps: float = 1e-5
    rope_theta: float = 1e6
    max_position_embeddings: int = 128_000
    conv_L_cache: int = 3               # taps of the short conv; its state keeps conv_L_cache - 1 inputs
    conv_bias: bool = False
    num_dense_layers: int = 2
    num_experts: int = 32
    num_experts_per_tok: int = 4
    routed_scaling_factor: float = 1.0
    use_expert_bias: bool = True
    norm_topk_prob: bool = True
    tie_word_embeddings: bool = True
    eos_token_id: int = 0
    bos_token_id: int | None = None
    pad_token_id: int | None = None
    eos_token_ids: list[int] = field(default_factory=list)
    path: str = ""

    # ---- derived (engine/models/lfm2_moe/config.py:84-123) ----
    @property
    def conv_state_len(self) -> int:
        return self.conv_L_cache - 1

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def is_attention(self, layer: int) -> bool:
        return self.layer_types[layer] == "full_attention"

    def is_moe(self, layer: int) -> bool:
        return layer >= self.num_dense_layers

    @property
    def attention_layers(self) -> list[int]:
        return [i for i, t in enumerate(self.layer_types) if t == "full_attention"]

    @property
    def conv_layers(self) -> list[int]:
        return [i for i, t in enumerate(self.layer_types) if t == "conv"]

    def kv_bytes_per_token(self, elem: int = 2) -> int:
        return len(self.attention_layers) * 2 * self.kv_dim * elem

    def conv_state_bytes(self, elem: int = 4) -> int:
        return len(self.conv_layers) * self.conv_state_len * self.hidden_size * elem

    # ---- config.json out and in ----
    def to_dict(self) -> dict:
        """The config.json of this configuration (the keys `from_dict` reads)."""
        d = asdict(self)
        d.pop("path")
        d.pop("eos_token_ids")
        theta = d.pop("rope_theta")
        d["rope_parameters"] = {"rope_theta": theta, "rope_type": "default"}
        d["model_type"] = MODEL_TYPES[0]
        d["architectures"] = [ARCHITECTURES[0]]
        return d

    @classmethod
    def from_dict(cls, raw: dict, path: str = "", generation: dict | None = None) -> "Lfm2MoeConfig":
        t = raw.get("text_config") or raw
        _check_keys(t)
        for key in ("hidden_size", "intermediate_size", "moe_intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "vocab_size"):
            if key not in t:
                raise ValueError(f"LFM2 MoE config lacks the required key {key!r}")
        n = int(t["num_hidden_layers"])
        layer_types = t.get("layer_types")
        if layer_types is None:
            # checkpoints that list their attention layers by index (engine/models/lfm2_moe/config.py:129-133)
            idx = set(t.get("full_attn_idxs") or [])
            layer_types = ["full_attention" if i in idx else "conv" for i in range(n)]
        rope = t.get("rope_parameters") or {}
        if rope.get("rope_type", "default") != "default":
            raise ValueError(f"LFM2 MoE rope_type {rope.get('rope_type')!r}: only 'default' is implemented")
        eos = t.get("eos_token_id", raw.get("eos_token_id"))
        eos_list = list(eos) if isinstance(eos, (list, tuple)) else ([] if eos is None else [eos])
        if not eos_list:
            raise ValueError("LFM2 MoE config lacks the required key 'eos_token_id'")
        stop = []
        if generation:
            g = generation.get("eos_token_id")
            stop = list(g) if isinstance(g, (list, tuple)) else ([] if g is None else [g])
        tie = t.get("tie_word_embeddings", t.get("tie_embedding", True))
        hidden = int(t["hidden_size"])
        heads = int(t["num_attention_heads"])
        cfg = cls(
            hidden_size=hidden,
            intermediate_size=int(t["intermediate_size"]),
            moe_intermediate_size=int(t["moe_intermediate_size"]),
            num_hidden_layers=n,
            num_attention_heads=heads,
            num_key_value_heads=int(t.get("num_key_value_heads", heads)),
            head_dim=int(t.get("head_dim") or hidden // heads),
            vocab_size=int(t["vocab_size"]),
            layer_types=[str(x) for x in layer_types],
            norm_eps=float(t.get("norm_eps", 1e-5)),
            rope_theta=float(rope.get("rope_theta", t.get("rope_theta", 1e6))),
            max_position_embeddings=int(t.get("max_position_embeddings", 128_000)),
            conv_L_cache=int(t.get("conv_L_cache", 3)),
            conv_bias=bool(t.get("conv_bias", False)),
            num_dense_layers=int(t.get("num_dense_layers", 2)),
            num_experts=int(t.get("num_experts", 32)),
            num_experts_per_tok=int(t.get("num_experts_per_tok", 4)),
            routed_scaling_factor=float(t.get("routed_scaling_factor", 1.0)),
            use_expert_bias=bool(t.get("use_expert_bias", True)),
            norm_topk_prob=bool(t.get("norm_topk_prob", True)),
            tie_word_embeddings=bool(tie),
            eos_token_id=int(eos_list[0]),
            bos_token_id=t.get("bos_token_id"),
            pad_token_id=t.get("pad_token_id"),
            eos_token_ids=[int(x) for x in stop] or [int(x) for x in eos_list],
            path=path,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        c = self
        if len(c.layer_types) != c.num_hidden_layers or set(c.layer_types) - set(LAYER_KINDS):
            raise ValueError(f"layer_types must name conv or full_attention for each of {c.num_hidden_layers} layers")
        for key in ("hidden_size", "intermediate_size", "moe_intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "vocab_size", "num_experts"):
            if getattr(c, key) <= 0:
                raise ValueError(f"{key} must be positive, got {getattr(c, key)}")
        if c.num_attention_heads % c.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if c.head_dim % 2:
            raise ValueError("the rotary position encoding needs an even head_dim")
        if not 0 < c.num_experts_per_tok <= c.num_experts:
            raise ValueError("num_experts_per_tok must be in 1..num_experts")
        if not 0 <= c.num_dense_layers <= c.num_hidden_layers:
            raise ValueError("num_dense_layers must be in 0..num_hidden_layers")
        if c.conv_L_cache < 2:
            raise ValueError("conv_L_cache must be at least 2")
        if not c.norm_eps > 0 or not c.rope_theta > 0:
            raise ValueError("norm_eps and rope_theta must be positive")

    # ---- the architecture-neutral form ----
    def to_spec(self) -> ModelSpec:
        c = self
        norm = PartSpec("rmsnorm", {"eps": c.norm_eps})
        attention = PartSpec("attention", {
            "num_heads": c.num_attention_heads, "num_kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
            "qk_norm": PartSpec("rmsnorm", {"eps": c.norm_eps}),
            "position": PartSpec("rope_neox", {"theta": c.rope_theta, "rotary_dim": c.head_dim}),
            "scale": c.head_dim ** -0.5, "window": None,
            "names": {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj",
                      "out": "self_attn.out_proj", "q_norm": "self_attn.q_layernorm",
                      "k_norm": "self_attn.k_layernorm"},
        })
        conv = PartSpec("short_conv", {
            "taps": c.conv_L_cache, "bias": c.conv_bias,
            "names": {"in": "conv.in_proj", "taps": "conv.conv", "out": "conv.out_proj"},
        })
        dense = PartSpec("swiglu", {
            "intermediate_size": c.intermediate_size,
            "names": {"gate": "feed_forward.w1", "up": "feed_forward.w3", "down": "feed_forward.w2"},
        })
        experts = PartSpec("sigmoid_topk_experts", {
            "num_experts": c.num_experts, "top_k": c.num_experts_per_tok,
            "intermediate_size": c.moe_intermediate_size, "expert_bias": c.use_expert_bias,
            "normalize": c.norm_topk_prob, "scale": c.routed_scaling_factor, "norm_floor": 1e-6,
            "names": {"router": "feed_forward.gate", "bias": "feed_forward.expert_bias",
                      "experts": "feed_forward.experts", "gate": "w1", "up": "w3", "down": "w2"},
        })
        layers = tuple(
            LayerSpec(prefix=f"layers.{i}.",
                      mixer=attention if c.is_attention(i) else conv,
                      feed_forward=experts if c.is_moe(i) else dense,
                      mixer_norm=PartSpec("rmsnorm", {"eps": c.norm_eps, "name": "operator_norm"}),
                      feed_forward_norm=PartSpec("rmsnorm", {"eps": c.norm_eps, "name": "ffn_norm"}))
            for i in range(c.num_hidden_layers))
        return ModelSpec(
            architecture=ARCHITECTURES[0], hidden_size=c.hidden_size, vocab_size=c.vocab_size,
            layers=layers, schedule=plain_schedule(c.num_hidden_layers), final_norm=norm,
            embedding_name="embed_tokens.weight", final_norm_prefix="embedding_norm.",
            head_name=None if c.tie_word_embeddings else "lm_head.weight",
            # a tied checkpoint may still store a copy of the head (the reference reads it when given,
            # engine/models/lfm2_moe/ref.py:96-97; here the tied model ignores it)
            ignored_names=("lm_head.weight",) if c.tie_word_embeddings else (),
            max_positions=c.max_position_embeddings, stop_token_ids=tuple(c.eos_token_ids),
        )


def _check_keys(t: dict) -> None:
    unknown = sorted(set(t) - KNOWN - IGNORED - set(FIXED))
    if unknown:
        raise ValueError(f"LFM2 MoE config key(s) this engine does not know: {', '.join(unknown)}")
    for key, want in FIXED.items():
        if key in t and t[key] != want:
            raise ValueError(f"LFM2 MoE config {key}={t[key]!r}: only {want!r} is implemented")


def load_config(folder: str) -> Lfm2MoeConfig:
    """The configuration of a model folder (config.json, and generation_config.json's stop ids if present)."""
    with open(os.path.join(folder, "config.json")) as f:
        raw = json.load(f)
    generation = None
    gpath = os.path.join(folder, "generation_config.json")
    if os.path.isfile(gpath):
        with open(gpath) as f:
            generation = json.load(f)
    return Lfm2MoeConfig.from_dict(raw, folder, generation)
