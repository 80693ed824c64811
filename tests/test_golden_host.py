"""The engine's host side against what the reference's own code says, recorded in
tests/golden/golden.json by tests/golden/make_golden.py: its ``parse_config`` on the real-M3-shaped
config.json of its tests (raw and native key shapes), the names, shapes and dtypes of the state dict
its ``create_model`` builds on the meta device, and the page accounting of its managers under the
chunked-prefill drive of its regression test."""

from __future__ import annotations

import json
import os

import pytest
import torch

from freetoken_b200.cache import CacheManager
from freetoken_b200.config.minimax_m3 import FFN_MOE, MIXER_SPARSE, MiniMaxM3Config
from freetoken_b200.config.spec import PagedKVNeed
from freetoken_b200.engine.build import describe_model


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("shape", ["raw", "native"])
def test_config_reader_agrees_with_the_reference_on_the_real_model(golden, shape):
    """python/freetoken/models/minimax_m3/config.py:61-198 on the dict of
    tests/models/test_minimax_m3.py:27-79 (and its native re-spelling, :82-109)."""
    want = golden["config"]["parsed"]
    cfg = MiniMaxM3Config.from_dict(golden["config"][shape])
    got = {
        "num_layers": cfg.num_hidden_layers, "hidden_size": cfg.hidden_size, "num_qo_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "vocab_size": cfg.vocab_size,
        "rotary_dim": cfg.rotary_dim, "rope_theta": cfg.rope_theta, "max_position": cfg.max_position_embeddings,
        "rms_norm_eps": cfg.rms_norm_eps, "hidden_act": cfg.hidden_act, "swiglu_alpha": cfg.swiglu_alpha,
        "swiglu_limit": cfg.swiglu_limit, "num_experts": cfg.num_local_experts,
        "num_experts_per_tok": cfg.num_experts_per_tok, "moe_intermediate_size": cfg.intermediate_size,
        "dense_intermediate_size": cfg.dense_intermediate_size,
        "shared_intermediate_size": cfg.shared_intermediate_size, "n_shared_experts": cfg.n_shared_experts,
        "routed_scaling_factor": cfg.routed_scaling_factor, "tie_word_embeddings": cfg.tie_word_embeddings,
        "moe_layer_ids": [l for l, t in enumerate(cfg.ffn_types) if t == FFN_MOE],
        "sparse_layer_ids": [l for l, t in enumerate(cfg.mixer_types) if t == MIXER_SPARSE],
        "index_dim": cfg.sparse.index_dim, "num_index_heads": cfg.sparse.num_index_heads,
        "topk_blocks": cfg.sparse.topk_blocks, "block_size": cfg.sparse.block_size,
        "init_blocks": cfg.sparse.init_blocks, "local_blocks": cfg.sparse.local_blocks,
    }
    assert got == want
    assert cfg.use_qk_norm and cfg.use_gemma_norm and cfg.scoring_func == "sigmoid" and cfg.use_routing_bias


def test_expected_tensors_are_the_reference_models_state_dict(golden):
    """Names, shapes and stored dtypes of every tensor, for three dense layers and two block-sparse MoE
    layers of the real sizes (python/freetoken/models/minimax_m3/model.py:25-97 built by
    ``create_model`` on the meta device in bfloat16).  The router matrix and its bias are 32-bit there
    too (moe.py:44-49)."""
    raw = golden["state_dict"]["config"]
    _, _, spec, expected = describe_model(raw)
    want = golden["state_dict"]["tensors"]
    assert sorted(expected) == sorted(want)
    for name, ps in expected.items():
        shape, dtype = want[name]
        assert list(ps.shape) == shape, name
        assert ps.storage_dtype() == dtype, name
    assert len(spec.layers) == 5 and [ls.ffn.kind for ls in spec.layers] == ["gated_mlp"] * 3 + ["moe"] * 2


def test_page_accounting_under_the_references_chunked_prefill_drive(golden):
    """tests/scheduler/test_scheduler_chunked_prefill.py:49-90 run on the reference's managers with its
    cache type that keeps nothing after a request: a prompt fed in portions takes its pages portion by
    portion, nothing is freed twice, everything is back at the end."""
    need = PagedKVNeed((("k", 1, 8), ("v", 1, 8)))
    for case in golden["chunked_prefill"]:
        m = CacheManager([(0, need)], 1, case["pages"], 4, case["pages"], torch.float32, torch.device("cpu"),
                         max_step_tokens=case["chunk"])
        m.open(7)
        pool = m.paged[0].pool
        for it in case["trail"]:
            if it["scheduled"]:
                m.begin_step([(7, it["scheduled"])])
                m.end_step()
            m.check()
            assert pool.free_count == it["free"]
        assert m.length(7) == case["chunks"] * case["chunk"]
        m.close(7)
        m.check()
        assert pool.free_count == case["free_at_end"] == case["pages"]
