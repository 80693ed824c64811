"""Configuration: config.json keys -> typed config -> model description; the registry; errors."""

import copy

import pytest

from freetoken_b200.config.engine_config import EngineConfig
from freetoken_b200.config.minimax_m3 import MiniMaxM3Config
from freetoken_b200.engine.build import describe_model
from freetoken_b200.errors import ConfigError
from freetoken_b200.registry import get_architecture, known_architectures
from tiny_configs import ALL, TINY_A, TINY_B, TINY_C, TINY_D


def test_every_key_is_read():
    a = MiniMaxM3Config.from_dict(TINY_A)
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads) == (64, 2, 4, 2)
    assert (a.head_dim, a.rotary_dim, a.rope_theta, a.rms_norm_eps) == (16, 8, 10000.0, 1e-6)
    assert a.use_qk_norm and a.use_gemma_norm and not a.tie_word_embeddings
    assert (a.num_local_experts, a.num_experts_per_tok, a.intermediate_size) == (8, 2, 32)
    assert a.scoring_func == "sigmoid" and a.use_routing_bias and a.hidden_act == "silu"
    assert a.ffn_types == ("moe", "moe") and a.mixer_types == ("full", "full")
    b = MiniMaxM3Config.from_dict(TINY_B)
    assert (b.head_dim, b.rotary_dim, b.rope_theta, b.rms_norm_eps) == (32, 32, 1e6, 1e-5)
    assert not b.use_qk_norm and not b.use_gemma_norm and b.tie_word_embeddings
    assert b.scoring_func == "softmax" and not b.use_routing_bias


def test_wrapper_defaults_and_native_key_shape():
    c = MiniMaxM3Config.from_dict(TINY_C)
    assert c.wrapped and c.rotary_dim == 24  # head_dim 48 * partial_rotary_factor 0.5
    assert c.ffn_types == ("dense", "moe", "moe") and c.dense_intermediate_size == 72
    assert c.n_shared_experts == 1 and c.shared_intermediate_size == 24 and c.routed_scaling_factor == 2.0
    native = copy.deepcopy(TINY_A)
    del native["rope_theta"]
    native["rope_parameters"] = {"rope_theta": 123.0, "rope_type": "default"}
    native["mlp_layer_types"] = ["dense", "sparse"]
    native["layer_types"] = ["full_attention", "minimax_m3_sparse"]
    native.update(index_n_heads=2, index_head_dim=16, index_block_size=8, index_topk_blocks=2, index_local_blocks=1)
    n = MiniMaxM3Config.from_dict(native)
    assert n.rope_theta == 123.0 and n.ffn_types == ("dense", "moe") and n.mixer_types == ("full", "sparse")
    assert n.sparse.block_size == 8 and n.sparse.topk_blocks == 2
    d = MiniMaxM3Config.from_dict(TINY_D)
    assert d.mixer_types == ("full", "sparse", "sparse") and d.sparse.index_dim == 16


def test_round_trip_and_layer_cap():
    for raw in ALL.values():
        cfg = MiniMaxM3Config.from_dict(raw)
        again = MiniMaxM3Config.from_dict(cfg.to_dict())
        for f in ("hidden_size", "head_dim", "rotary_dim", "ffn_types", "mixer_types", "scoring_func",
                  "hidden_act", "routed_scaling_factor", "n_shared_experts", "tie_word_embeddings"):
            assert getattr(cfg, f) == getattr(again, f), f
    assert MiniMaxM3Config.from_dict(TINY_B, num_layers=2).num_hidden_layers == 2


@pytest.mark.parametrize("key,value", [
    ("scoring_func", "tanh"), ("hidden_act", "gelu"), ("qk_norm_type", "per_layer"),
    ("attention_output_gate", True), ("swiglu_beta", 2.0), ("rope_scaling", {"rope_type": "yarn"}),
    ("num_key_value_heads", 3), ("rotary_dim", 18), ("num_experts_per_tok", 9), ("hidden_size", 0),
    ("attn_type_list", [0, 1])])
def test_unsupported_values_name_their_key(key, value):
    raw = dict(TINY_A, **{key: value})
    with pytest.raises(ConfigError) as e:
        MiniMaxM3Config.from_dict(raw)
    assert key.split("_")[0] in str(e.value)


def test_missing_key_and_sparse_checks():
    raw = dict(TINY_A)
    del raw["rms_norm_eps"]
    with pytest.raises(ConfigError, match="rms_norm_eps"):
        MiniMaxM3Config.from_dict(raw)
    bad = copy.deepcopy(TINY_D)
    bad["sparse_attention_config"]["sparse_index_dim"] = 32
    with pytest.raises(ConfigError, match="sparse_index_dim"):
        MiniMaxM3Config.from_dict(bad)
    bad = copy.deepcopy(TINY_D)
    bad["sparse_attention_config"]["sparse_topk_blocks"] = 64
    with pytest.raises(ConfigError, match="sparse_topk_blocks"):
        MiniMaxM3Config.from_dict(bad)


def test_registry_and_model_description():
    assert "MiniMaxM3SparseForCausalLM" in known_architectures()
    assert get_architecture("MiniMaxM3SparseForConditionalGeneration") is get_architecture("MiniMaxM3SparseForCausalLM")
    with pytest.raises(ConfigError, match="not supported"):
        get_architecture("LlamaForCausalLM")
    arch, typed, spec, expected = describe_model(TINY_C)
    assert [l.ffn.kind for l in spec.layers] == ["gated_mlp", "moe", "moe"]
    assert [l.ffn_name for l in spec.layers] == ["mlp", "block_sparse_moe", "block_sparse_moe"]
    assert expected["model.layers.1.block_sparse_moe.gate.weight"].dtype == "float32"
    assert expected["model.layers.1.block_sparse_moe.experts.gate_up_proj"].shape == (6, 80, 112)
    assert expected["model.layers.1.block_sparse_moe.shared_experts.gate_up_proj.weight"].shape == (48, 112)
    assert expected["model.layers.0.mlp.down_proj.weight"].shape == (112, 72)
    assert expected["model.layers.0.self_attn.qkv_proj.weight"].shape == ((7 + 2) * 48, 112)
    assert "lm_head.weight" in expected
    _, _, spec_b, exp_b = describe_model(TINY_B)
    assert "lm_head.weight" not in exp_b and "model.layers.0.self_attn.q_norm.weight" not in exp_b
    assert [e.layer for e in spec_b.schedule] == [0, 1, 2]


def test_engine_config_checks():
    with pytest.raises(ConfigError):
        EngineConfig(model_path="x", dtype="float16")
    with pytest.raises(ConfigError):
        EngineConfig(model_path="x", page_size=0)
    with pytest.raises(ConfigError):
        EngineConfig(model_path="x", num_token_override=10, page_size=4)
    assert EngineConfig(model_path="x", num_token_override=64, page_size=16).num_page_override == 4
    assert EngineConfig(model_path="x", dtype="bf16").dtype == "bfloat16"
