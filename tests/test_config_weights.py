"""Configuration, registry, and weight loading errors (no device needed)."""

import json
import os

import pytest
import torch

from tandemllm_b200.config import (Architecture, Lfm2MoeConfig, ModelSpec, PartSpec, Site, architecture_of,
                                   read_model_config, register, unregister)
from tandemllm_b200.config.spec import LayerSpec
from tandemllm_b200.parts.model import DecoderModel
from tandemllm_b200.weights.loader import DictWeights, FolderWeights
from tandemllm_b200.weights.random_init import write_model_folder
from tandemllm_b200.weights.safetensors_io import CheckpointError, index_folder, read_tensor, write_file
from tests import tiny_configs as T
from tests.helpers import random_model_weights, write_folder


def test_reads_every_key_and_derives_sizes():
    c = Lfm2MoeConfig.from_dict(T.TINY_B)
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (96, 3, 1, 32)
    assert (c.conv_L_cache, c.conv_bias, c.num_dense_layers, c.num_experts, c.num_experts_per_tok) == (4, True, 2, 8, 3)
    assert (c.norm_eps, c.rope_theta, c.routed_scaling_factor) == (1e-6, 1e6, 1.5)
    assert not c.use_expert_bias and not c.norm_topk_prob and not c.tie_word_embeddings
    assert c.attention_layers == [2, 4, 5] and c.conv_layers == [0, 1, 3]
    assert c.q_dim == 96 and c.kv_dim == 32 and c.conv_state_len == 3
    assert c.kv_bytes_per_token(2) == 3 * 2 * 32 * 2
    spec = c.to_spec()
    assert spec.head_name == "lm_head.weight" and len(spec.layers) == 6 and spec.stop_token_ids == (3,)
    assert spec.layers[2].mixer.kind == "attention" and spec.layers[0].mixer.kind == "short_conv"
    assert spec.layers[1].feed_forward.kind == "swiglu" and spec.layers[2].feed_forward.kind == "sigmoid_topk_experts"
    # round trip through config.json's form
    assert Lfm2MoeConfig.from_dict(c.to_dict()).to_spec() == spec


def test_defaults_and_fallbacks():
    raw = {k: v for k, v in T.TINY_A.items() if k not in ("layer_types", "head_dim", "num_key_value_heads", "rope_parameters")}
    raw["full_attn_idxs"] = [1, 3]
    raw["rope_theta"] = 5e5
    c = Lfm2MoeConfig.from_dict(raw)
    assert c.layer_types == ["conv", "full_attention", "conv", "full_attention"]
    assert c.head_dim == 16 and c.num_key_value_heads == 4 and c.rope_theta == 5e5
    gen = Lfm2MoeConfig.from_dict(T.TINY_A, generation={"eos_token_id": [2, 7]})
    assert gen.eos_token_ids == [2, 7] and gen.eos_token_id == 2


@pytest.mark.parametrize("change,needle", [
    ({"shiny_new_switch": 1}, "shiny_new_switch"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"quantization_config": {"bits": 4}}, "quantization_config"),
    ({"rope_parameters": {"rope_type": "yarn", "rope_theta": 1e6}}, "rope_type"),
    ({"layer_types": ["conv"] * 3}, "layer_types"),
    ({"layer_types": ["conv", "mamba", "conv", "conv"]}, "layer_types"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"num_experts_per_tok": 9}, "num_experts_per_tok"),
    ({"num_dense_layers": 9}, "num_dense_layers"),
    ({"conv_L_cache": 1}, "conv_L_cache"),
    ({"eos_token_id": None}, "eos_token_id"),
])
def test_bad_configs_are_refused_by_name(change, needle):
    with pytest.raises(ValueError, match=needle):
        Lfm2MoeConfig.from_dict({**T.TINY_A, **change})


def test_missing_required_key():
    raw = dict(T.TINY_A)
    del raw["moe_intermediate_size"]
    with pytest.raises(ValueError, match="moe_intermediate_size"):
        Lfm2MoeConfig.from_dict(raw)


def test_registry_selects_by_architecture_then_model_type():
    assert architecture_of(T.TINY_A).name == "lfm2_moe"
    assert architecture_of({"model_type": "lfm2_moe"}).name == "lfm2_moe"
    assert architecture_of({"text_config": {"model_type": "lfm2_moe"}}).name == "lfm2_moe"
    with pytest.raises(ValueError, match="lfm2_moe"):
        architecture_of({"architectures": ["SomethingElseForCausalLM"]})


def test_registering_another_architecture(tmp_path):
    def read(raw, folder, generation):
        norm = PartSpec("rmsnorm", {"eps": raw["eps"]})
        layer = LayerSpec("blocks.0.", PartSpec("short_conv", {"taps": 2, "names": {"in": "a", "taps": "b", "out": "c"}}),
                          PartSpec("swiglu", {"intermediate_size": 32, "names": {"gate": "g", "up": "u", "down": "d"}}),
                          PartSpec("rmsnorm", {"eps": raw["eps"], "name": "n1"}), PartSpec("rmsnorm", {"eps": raw["eps"], "name": "n2"}))
        return ModelSpec("ToyForCausalLM", 16, 40, (layer,), (Site(0), Site(0)), norm, embedding_name="tok.weight",
                         final_norm_prefix="last_norm.")
    register(Architecture("toy", ("ToyForCausalLM",), ("toy",), read))
    try:
        (tmp_path / "config.json").write_text(json.dumps({"architectures": ["ToyForCausalLM"], "eps": 1e-5}))
        arch, spec = read_model_config(str(tmp_path))
        assert arch.name == "toy" and len(spec.schedule) == 2
        names = [s.name for s in DecoderModel(spec).weight_specs()]
        assert "blocks.0.a.weight" in names and "blocks.0.n1.weight" in names and "last_norm.weight" in names and "tok.weight" in names
    finally:
        unregister("toy")


def test_schedule_is_checked():
    norm = PartSpec("rmsnorm", {"eps": 1e-5})
    names = dict(embedding_name="e.weight", final_norm_prefix="n.")
    with pytest.raises(ValueError, match="not before"):
        ModelSpec("X", 8, 8, (None,), (Site(0), Site(0, cache_of=1)), norm, **names)
    with pytest.raises(ValueError, match="names layer"):
        ModelSpec("X", 8, 8, (None,), (Site(1),), norm, **names)
    with pytest.raises(TypeError, match="embedding_name"):      # an architecture names its own tensors: no default
        ModelSpec("X", 8, 8, (None,), (Site(0),), norm)


# ------------------------------------------------------------------------------------------ weights
def test_random_folder_round_trip(tmp_path):
    c = Lfm2MoeConfig.from_dict(T.TINY_A)
    folder = write_model_folder(c, str(tmp_path / "m"), seed=5, std=0.02)
    again = write_model_folder(c, str(tmp_path / "m2"), seed=5, std=0.02)
    other = write_model_folder(c, str(tmp_path / "m3"), seed=6, std=0.02)
    a, b, o = (index_folder(f) for f in (folder, again, other))
    assert set(a) == set(b) and "model.embed_tokens.weight" in a and "model.layers.1.self_attn.q_layernorm.weight" in a
    key = "model.layers.2.feed_forward.experts.3.w2.weight"
    assert torch.equal(read_tensor(a[key]), read_tensor(b[key])) and not torch.equal(read_tensor(a[key]), read_tensor(o[key]))
    assert a[key].dtype == "BF16" and a["model.layers.1.feed_forward.expert_bias"].dtype == "F32"
    arch, cfg = read_model_config(folder)
    assert cfg.to_spec() == c.to_spec()
    fw = FolderWeights(folder)
    model = DecoderModel(cfg.to_spec())
    fw.check(model.weight_specs(fw.present()))
    assert fw.read("embed_tokens.weight").dtype == torch.bfloat16
    assert fw.read("layers.1.feed_forward.expert_bias").dtype == torch.float32
    w = read_tensor(a["model.embed_tokens.weight"]).float()
    assert abs(float(w.std()) - 0.02) < 0.002


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    W = random_model_weights(T.TINY_A, 0, 0.02)
    del W["layers.1.self_attn.k_layernorm.weight"]
    del W["layers.3.feed_forward.experts.2.w3.weight"]
    W["layers.0.conv.surprise"] = torch.zeros(3)
    W["layers.0.conv.in_proj.weight"] = torch.zeros(64, 192)
    folder = write_folder(str(tmp_path / "bad"), T.TINY_A, W)
    fw = FolderWeights(folder)
    model = DecoderModel(Lfm2MoeConfig.from_dict(T.TINY_A).to_spec())
    with pytest.raises(CheckpointError) as e:
        fw.check(model.weight_specs(fw.present()))
    msg = str(e.value)
    for needle in ("missing (2)", "layers.1.self_attn.k_layernorm.weight", "layers.3.feed_forward.experts.2.w3.weight",
                   "unexpected (1)", "layers.0.conv.surprise", "wrong shape (1)", "layers.0.conv.in_proj.weight",
                   "[64, 192]", "[192, 64]"):
        assert needle in msg, needle


def test_untied_head_must_be_present_and_tied_copy_is_ignored():
    Wb = random_model_weights(T.TINY_B, 1, 0.05)
    spec_b = Lfm2MoeConfig.from_dict(T.TINY_B).to_spec()
    missing = {k: v for k, v in Wb.items() if k != "lm_head.weight"}
    with pytest.raises(CheckpointError, match="lm_head.weight"):
        DictWeights(missing).check(DecoderModel(spec_b).weight_specs(set(missing)))
    Wa = random_model_weights(T.TINY_A, 0, 0.02)
    Wa["lm_head.weight"] = Wa["embed_tokens.weight"].clone()
    model = DecoderModel(Lfm2MoeConfig.from_dict(T.TINY_A).to_spec())
    DictWeights(Wa).check(model.weight_specs(set(Wa)), ignore=lambda n: n == "lm_head.weight")


def test_stacked_experts_are_accepted():
    W = random_model_weights(T.TINY_A, 0, 0.02)
    for li in (1, 2, 3):
        f = f"layers.{li}.feed_forward.experts."
        W[f + "gate_up_proj"] = torch.stack([torch.cat([W.pop(f + f"{e}.w1.weight"), W.pop(f + f"{e}.w3.weight")]) for e in range(4)])
        W[f + "down_proj"] = torch.stack([W.pop(f + f"{e}.w2.weight") for e in range(4)])
    model = DecoderModel(Lfm2MoeConfig.from_dict(T.TINY_A).to_spec())
    DictWeights(W).check(model.weight_specs(set(W)))


def test_file_errors_name_the_file(tmp_path):
    folder = tmp_path / "m"
    folder.mkdir()
    with pytest.raises(CheckpointError, match="neither"):
        index_folder(str(folder))
    write_file(str(folder / "model.safetensors"), {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3)})
    st = index_folder(str(folder))["a"]
    assert torch.equal(read_tensor(st), torch.arange(6.).reshape(2, 3))
    raw = (folder / "model.safetensors").read_bytes()
    (folder / "model.safetensors").write_bytes(raw[:-5])
    with pytest.raises(CheckpointError, match="truncated"):
        index_folder(str(folder))
    (folder / "model.safetensors").unlink()
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "part-1.safetensors"}}))
    with pytest.raises(CheckpointError, match="part-1.safetensors"):
        index_folder(str(folder))
    write_file(str(folder / "part-1.safetensors"), {"b": torch.zeros(2)})
    with pytest.raises(CheckpointError, match="no shard holds"):
        index_folder(str(folder))


def test_integer_tables_become_int32_and_32bit_stays(tmp_path):
    write_file(str(tmp_path / "model.safetensors"),
               {"t": torch.arange(4, dtype=torch.int64), "f": torch.ones(2, dtype=torch.float32),
                "h": torch.ones(2, dtype=torch.float16), "b": torch.ones(2, dtype=torch.bfloat16)})
    fw = FolderWeights(str(tmp_path), prefixes=("model.",))
    assert fw.read("t").dtype == torch.int32 and fw.read("f").dtype == torch.float32
    assert fw.read("h").dtype == torch.bfloat16 and fw.read("b").dtype == torch.bfloat16
