"""Tiny MiniMax-M3 configurations for tests; they differ in every size and option.

A: 2 layers, hidden 64, 4 q / 2 kv heads, head 16, partial rotary 8, theta 1e4, QK norm,
   8 experts top-2 width 32, sigmoid + bias, vocab 256, eps 1e-6, untied head.
B: 3 layers, hidden 96, 6 q / 3 kv heads, head 32, full rotary, theta 1e6, no QK norm,
   16 experts top-4 width 48, softmax without bias, vocab 384, eps 1e-5, tied head.
C: the reference's real options on small sizes: swigluoai, one dense prefix layer, a shared
   expert, routed_scaling_factor 2, 7 q / 1 kv heads of 48 (no power of two anywhere).
D: block-sparse attention layers after one full layer (index heads, 8-token blocks, top-3), two
   experts that every token uses.
E: A with 6 q / 2 kv heads of 128 and pages of 16 tokens: long steps run the tensor-core attention.
"""

from __future__ import annotations

import copy

ARCH = "MiniMaxM3SparseForCausalLM"

TINY_A = {
    "architectures": [ARCH], "model_type": "minimax_m3",
    "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "rotary_dim": 8,
    "rope_theta": 10000.0, "max_position_embeddings": 512, "rms_norm_eps": 1e-6,
    "use_qk_norm": True, "use_gemma_norm": True, "tie_word_embeddings": False,
    "hidden_act": "silu", "num_local_experts": 8, "num_experts_per_tok": 2,
    "intermediate_size": 32, "scoring_func": "sigmoid", "use_routing_bias": True,
    "routed_scaling_factor": 1.0, "n_shared_experts": 0, "torch_dtype": "bfloat16",
}

TINY_B = {
    "architectures": [ARCH], "model_type": "minimax_m3",
    "vocab_size": 384, "hidden_size": 96, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32, "rotary_dim": 32,
    "rope_theta": 1000000.0, "max_position_embeddings": 512, "rms_norm_eps": 1e-5,
    "use_qk_norm": False, "use_gemma_norm": False, "tie_word_embeddings": True,
    "hidden_act": "silu", "num_local_experts": 16, "num_experts_per_tok": 4,
    "intermediate_size": 48, "scoring_func": "softmax", "use_routing_bias": False,
    "routed_scaling_factor": 1.0, "n_shared_experts": 0, "torch_dtype": "bfloat16",
}

TINY_C = {
    "architectures": ["MiniMaxM3SparseForConditionalGeneration"], "model_type": "minimax_m3_vl",
    "text_config": {
        "vocab_size": 331, "hidden_size": 112, "num_hidden_layers": 3,
        "num_attention_heads": 7, "num_key_value_heads": 1, "head_dim": 48,
        "partial_rotary_factor": 0.5, "rope_theta": 5000000.0, "max_position_embeddings": 512,
        "rms_norm_eps": 1e-6, "use_qk_norm": True, "use_gemma_norm": True,
        "hidden_act": "swigluoai", "swiglu_alpha": 1.702, "swiglu_limit": 7.0,
        "num_local_experts": 6, "num_experts_per_tok": 3, "intermediate_size": 40,
        "dense_intermediate_size": 72, "shared_intermediate_size": 24, "n_shared_experts": 1,
        "moe_layer_freq": [0, 1, 1], "scoring_func": "sigmoid", "use_routing_bias": True,
        "routed_scaling_factor": 2.0, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
    },
}

TINY_D = dict(copy.deepcopy(TINY_A), **{
    "num_hidden_layers": 3,
    # every token uses both experts: the only discrete choice left is the choice of key blocks, so
    # bfloat16 runs can be compared over long stretches
    "num_local_experts": 2, "num_experts_per_tok": 2,
    "sparse_attention_config": {
        "use_sparse_attention": True, "sparse_attention_freq": [0, 1, 1],
        "sparse_num_index_heads": 2, "sparse_index_dim": 16, "sparse_block_size": 8,
        "sparse_topk_blocks": 3, "sparse_local_block": 1, "sparse_init_block": 0,
        "sparse_score_type": "max", "sparse_disable_index_value": [1, 1, 1],
    },
})

# E: heads of 128 with 3 query heads per KV head and pages of 16, the sizes the tensor-core attention
# kernel takes; everything else small.
TINY_E = dict(copy.deepcopy(TINY_A), **{
    "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128, "rotary_dim": 64,
    "max_position_embeddings": 1024, "num_local_experts": 4, "num_experts_per_tok": 2, "intermediate_size": 48,
})

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}
