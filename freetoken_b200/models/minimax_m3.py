"""MiniMax-M3: from its typed config to a model description, and its checkpoint names.

Layer structure (python/freetoken/models/minimax_m3/model.py:25-97): pre-norm residual
layers, attention under ``self_attn``, the feed-forward under ``mlp`` (dense layers) or
``block_sparse_moe`` (MoE layers), every norm the Gemma (1+w) RMSNorm when
``use_gemma_norm`` is set.

Checkpoint names (python/freetoken/models/minimax_m3/weight.py:182-246,47-63): text tensors
may carry a ``language_model.`` prefix; ``q_proj``/``k_proj``/``v_proj`` are concatenated
along dim 0 into ``qkv_proj`` (:186-191); ``gate_proj``/``up_proj`` into ``gate_up_proj``
(:223-242); experts come one tensor per expert as ``experts.{e}.w1`` (gate), ``w3`` (up),
``w2`` (down) and are stacked into ``experts.gate_up_proj [E, 2I, H]`` and
``experts.down_proj [E, H, I]`` (python/freetoken/layers/moe.py:83-92).  Already fused
spellings are accepted as they are.
"""

from __future__ import annotations

from typing import Any, Dict, List, Mapping, Optional

from ..config.minimax_m3 import (ARCHITECTURES, FFN_MOE, MIXER_FULL, MIXER_SPARSE, MiniMaxM3Config)
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..errors import ConfigError
from ..registry import Architecture, register_architecture
from ..weights.binder import FusionRule


def build_spec(cfg: MiniMaxM3Config) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps, gemma=cfg.use_gemma_norm))
    position = PartSpec("rope_neox", dict(rotary_dim=cfg.rotary_dim, theta=cfg.rope_theta))
    block = PartSpec("prenorm_residual", dict(hidden=cfg.hidden_size, norm=norm))
    layers: List[LayerSpec] = []
    for l in range(cfg.num_hidden_layers):
        attn = dict(hidden=cfg.hidden_size, n_heads=cfg.num_attention_heads,
                    n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                    qk_norm=cfg.use_qk_norm, eps=cfg.rms_norm_eps, gemma=cfg.use_gemma_norm,
                    position=position, window=None)
        if cfg.mixer_types[l] == MIXER_FULL:
            mixer = PartSpec("gqa_attention", attn)
        elif cfg.mixer_types[l] == MIXER_SPARSE:
            sp = cfg.sparse
            mixer = PartSpec("block_sparse_attention", dict(
                attn, index_dim=sp.index_dim, n_index_heads=sp.num_index_heads,
                block_size=sp.block_size, topk_blocks=sp.topk_blocks,
                local_blocks=sp.local_blocks, init_blocks=sp.init_blocks))
        else:
            raise ConfigError(f"layer {l}: unknown mixer type '{cfg.mixer_types[l]}'")
        if cfg.ffn_types[l] == FFN_MOE:
            ffn = PartSpec("moe", dict(
                hidden=cfg.hidden_size, inter=cfg.intermediate_size, n_experts=cfg.num_local_experts,
                top_k=cfg.num_experts_per_tok, scoring=cfg.scoring_func, bias=cfg.use_routing_bias,
                scale=cfg.routed_scaling_factor, act=cfg.hidden_act, alpha=cfg.swiglu_alpha,
                limit=cfg.swiglu_limit,
                shared_inter=cfg.shared_intermediate_size * cfg.n_shared_experts))
            ffn_name = "block_sparse_moe"
        else:
            ffn = PartSpec("gated_mlp", dict(
                hidden=cfg.hidden_size, inter=cfg.dense_intermediate_size, act=cfg.hidden_act,
                alpha=cfg.swiglu_alpha, limit=cfg.swiglu_limit))
            ffn_name = "mlp"
        layers.append(LayerSpec(name=f"model.layers.{l}", block=block, mixer=mixer, ffn=ffn,
                                mixer_name="self_attn", ffn_name=ffn_name))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(l) for l in range(cfg.num_hidden_layers)),
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab_size, hidden=cfg.hidden_size)),
        final_norm=norm,
        head=PartSpec("linear_head", dict(tied=cfg.tie_word_embeddings)),
        max_position=cfg.max_position_embeddings,
        eos_token_ids=cfg.eos_token_ids,
        source=cfg,
    )


def fusion_rules(cfg: MiniMaxM3Config) -> List[FusionRule]:
    """How checkpoint tensors combine into the model's tensors."""
    rules: List[FusionRule] = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}"
        rules.append(FusionRule(f"{p}.self_attn.qkv_proj.weight",
                                [f"{p}.self_attn.{x}_proj.weight" for x in ("q", "k", "v")], "cat0",
                                [cfg.num_attention_heads * cfg.head_dim,
                                 cfg.num_key_value_heads * cfg.head_dim,
                                 cfg.num_key_value_heads * cfg.head_dim]))
        if cfg.mixer_types[l] == MIXER_SPARSE:
            rules.append(FusionRule(f"{p}.self_attn.index_qk_proj.weight",
                                    [f"{p}.self_attn.index_q_proj.weight",
                                     f"{p}.self_attn.index_k_proj.weight"], "cat0",
                                    [cfg.sparse.num_index_heads * cfg.sparse.index_dim,
                                     cfg.sparse.index_dim]))
        if cfg.ffn_types[l] == FFN_MOE:
            m = f"{p}.block_sparse_moe"
            E = cfg.num_local_experts
            rules.append(FusionRule(
                f"{m}.experts.gate_up_proj",
                [f"{m}.experts.{e}.{w}.weight" for e in range(E) for w in ("w1", "w3")],
                "stack_pairs"))
            rules.append(FusionRule(f"{m}.experts.down_proj",
                                    [f"{m}.experts.{e}.w2.weight" for e in range(E)], "stack"))
            if cfg.n_shared_experts:
                rules.append(FusionRule(f"{m}.shared_experts.gate_up_proj.weight",
                                        [f"{m}.shared_experts.gate_proj.weight",
                                         f"{m}.shared_experts.up_proj.weight"], "cat0"))
        else:
            rules.append(FusionRule(f"{p}.mlp.gate_up_proj.weight",
                                    [f"{p}.mlp.gate_proj.weight", f"{p}.mlp.up_proj.weight"], "cat0"))
    return rules


def parse(raw: Mapping[str, Any], num_layers: Optional[int] = None) -> MiniMaxM3Config:
    return MiniMaxM3Config.from_dict(raw, num_layers=num_layers)


def ignorable(name: str) -> bool:
    """Tensors of the checkpoint the text model never reads (weight.py:3-6), and the head of
    a tied model (python/freetoken/layers/embedding.py:81-90)."""
    return name.startswith(("vision_tower.", "multi_modal_projector.", "patch_merge_mlp."))


ARCH = Architecture(
    names=ARCHITECTURES,
    parse_config=parse,
    build_spec=build_spec,
    fusion_rules=fusion_rules,
    name_prefixes=("language_model.",),
    ignorable=ignorable,
)
register_architecture(ARCH)
