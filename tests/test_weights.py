"""Weights: safetensors I/O, binding by name, the one error that lists everything wrong."""

import json
import os

import pytest
import torch

from freetoken_b200.engine.build import describe_model
from freetoken_b200.errors import WeightError
from freetoken_b200.weights.binder import bind_folder
from freetoken_b200.weights.random_init import write_model_folder
from freetoken_b200.weights.safetensors_io import ModelFolder, write_safetensors
from tiny_configs import TINY_A, TINY_B, TINY_C

CPU = torch.device("cpu")


def bind(folder, raw, dtype=torch.bfloat16):
    arch, typed, spec, expected = describe_model(raw)
    optional = ("lm_head.weight",) if typed.tie_word_embeddings else ()
    return bind_folder(folder, expected, arch.fusion_rules(typed), dtype, CPU,
                       prefixes=arch.name_prefixes, ignorable=arch.ignorable, optional=optional), expected


def test_writer_matches_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file

    write_model_folder(TINY_A, str(tmp_path), seed=3)
    ours = ModelFolder(str(tmp_path))
    theirs = load_file(os.path.join(tmp_path, "model.safetensors"))
    assert sorted(ours.names()) == sorted(theirs)
    for n in theirs:
        assert torch.equal(ours.read(n), theirs[n])
    assert theirs["model.layers.0.block_sparse_moe.gate.weight"].dtype == torch.float32
    assert theirs["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert "model.layers.0.block_sparse_moe.experts.3.w1.weight" in theirs
    with open(os.path.join(tmp_path, "config.json")) as f:
        assert json.load(f)["hidden_size"] == 64


def test_same_seed_same_weights_and_dtypes(tmp_path):
    a, b, c = tmp_path / "a", tmp_path / "b", tmp_path / "c"
    write_model_folder(TINY_C, str(a), seed=5)
    write_model_folder(TINY_C, str(b), seed=5)
    write_model_folder(TINY_C, str(c), seed=6)
    ta, _ = bind(str(a), TINY_C)
    tb, _ = bind(str(b), TINY_C)
    tc, expected = bind(str(c), TINY_C)
    assert all(torch.equal(ta[n], tb[n]) for n in ta)
    assert any(not torch.equal(ta[n], tc[n]) for n in ta)
    assert set(ta) == set(expected)
    assert ta["model.layers.1.block_sparse_moe.gate.weight"].dtype == torch.float32
    assert ta["model.layers.1.block_sparse_moe.e_score_correction_bias"].dtype == torch.float32
    assert ta["model.norm.weight"].dtype == torch.float32
    assert ta["model.layers.1.block_sparse_moe.experts.gate_up_proj"].dtype == torch.bfloat16
    t32, _ = bind(str(a), TINY_C, torch.float32)
    assert t32["model.embed_tokens.weight"].dtype == torch.float32
    assert torch.equal(t32["model.embed_tokens.weight"], ta["model.embed_tokens.weight"].float())
    # norm scales ~ N(0, 0.02) in the Gemma form, router bias ~ N(0, 0.01)
    assert ta["model.norm.weight"].abs().max() < 0.2
    assert ta["model.layers.1.block_sparse_moe.e_score_correction_bias"].abs().max() < 0.1


def test_fusions_prefix_and_fused_spelling(tmp_path):
    from safetensors.torch import load_file, save_file

    split, fused, pref = tmp_path / "s", tmp_path / "f", tmp_path / "p"
    write_model_folder(TINY_C, str(split), seed=1)
    write_model_folder(TINY_C, str(fused), seed=1, fused_names=True)
    ts, _ = bind(str(split), TINY_C)
    tf, _ = bind(str(fused), TINY_C)
    assert all(torch.equal(ts[n], tf[n]) for n in ts)
    raw = load_file(os.path.join(split, "model.safetensors"))
    q, k, v = (raw[f"model.layers.0.self_attn.{x}_proj.weight"] for x in "qkv")
    assert torch.equal(ts["model.layers.0.self_attn.qkv_proj.weight"], torch.cat([q, k, v]))
    w1, w3 = (raw[f"model.layers.2.block_sparse_moe.experts.4.{w}.weight"] for w in ("w1", "w3"))
    assert torch.equal(ts["model.layers.2.block_sparse_moe.experts.gate_up_proj"][4], torch.cat([w1, w3]))
    os.makedirs(pref)
    save_file({"language_model." + n: t for n, t in raw.items()} |
              {"vision_tower.blocks.0.weight": torch.zeros(2)}, os.path.join(pref, "model.safetensors"))
    with open(os.path.join(pref, "config.json"), "w") as f:
        json.dump(TINY_C, f)
    tp, _ = bind(str(pref), TINY_C)
    assert all(torch.equal(ts[n], tp[n]) for n in ts)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from safetensors.torch import load_file, save_file

    write_model_folder(TINY_A, str(tmp_path), seed=1)
    path = os.path.join(tmp_path, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.self_attn.k_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.o_proj.weight"] = torch.zeros(64, 65, dtype=torch.bfloat16)
    t["model.layers.0.block_sparse_moe.experts.2.w2.weight"] = torch.zeros(64, 31, dtype=torch.bfloat16)
    t["model.layers.7.extra.weight"] = torch.zeros(3)
    t["model.embed_tokens.weight"] = torch.zeros(256, 64, dtype=torch.int32)
    save_file(t, path)
    with pytest.raises(WeightError) as e:
        bind(str(tmp_path), TINY_A)
    msg = str(e.value)
    assert "model.layers.1.self_attn.k_proj.weight" in msg and "model.norm.weight" in msg
    assert "model.layers.7.extra.weight" in msg
    assert "o_proj.weight: file has [64, 65], model expects [64, 64]" in msg
    assert "experts.2.w2.weight" in msg and "embed_tokens" in msg
    assert e.value.missing == ["model.layers.1.self_attn.k_proj.weight", "model.norm.weight"]
    assert e.value.unexpected == ["model.layers.7.extra.weight"]
    assert len(e.value.wrong) == 3


def test_tied_head_ignores_a_stray_lm_head(tmp_path):
    from safetensors.torch import load_file, save_file

    write_model_folder(TINY_B, str(tmp_path), seed=1)
    path = os.path.join(tmp_path, "model.safetensors")
    t = load_file(path)
    assert "lm_head.weight" not in t
    t["lm_head.weight"] = torch.zeros(384, 96, dtype=torch.bfloat16)
    save_file(t, path)
    bind(str(tmp_path), TINY_B)


def test_broken_files(tmp_path):
    with pytest.raises(WeightError, match="no .safetensors"):
        ModelFolder(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00garbage")
    with pytest.raises(WeightError):
        ModelFolder(str(tmp_path))
    good = tmp_path / "g"
    os.makedirs(good)
    write_safetensors(str(good / "model.safetensors"), {"a": torch.arange(6, dtype=torch.int32).view(2, 3)})
    assert torch.equal(ModelFolder(str(good)).read("a"), torch.arange(6, dtype=torch.int32).view(2, 3))
