"""Typed MiniMax-M3 configuration, read from the architecture's own config.json keys.

Key names, defaults and the rejected variants follow the reference's reader
(python/freetoken/models/minimax_m3/args.py:78-254 and config.py:61-198).  Both key
shapes are accepted: the raw checkpoint dict (``rope_theta``,
``sparse_attention_config``, ``moe_layer_freq``) and the native shape
(``rope_parameters``, ``layer_types`` / ``index_*``, ``mlp_layer_types``); a wrapper
config is unwrapped through ``text_config`` (config.py:42-43).  Every unsupported
variant the reference asserts on becomes a :class:`ConfigError` naming the key.

Options that the reference pins but this engine takes from config.json:
``use_qk_norm`` (false skips the per-head norms), ``use_gemma_norm`` (false multiplies
by ``w`` instead of ``1+w``), ``hidden_act`` (``"swigluoai"`` is the clamped form; ``"silu"`` is
plain SwiGLU unless ``swiglu_alpha`` / ``swiglu_limit`` stand beside it, which is how the native
key shape spells the clamped form), ``scoring_func`` (``"sigmoid"`` or ``"softmax"``),
``use_routing_bias``, ``n_shared_experts`` (0 means no shared expert) and
``attn_type_list`` as an alias for a per-layer mixer choice (0 = full attention).
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..errors import ConfigError
from .reader import read_config_json

ARCHITECTURES = ("MiniMaxM3SparseForCausalLM", "MiniMaxM3SparseForConditionalGeneration")

MIXER_FULL = "full"
MIXER_SPARSE = "sparse"
FFN_DENSE = "dense"
FFN_MOE = "moe"


@dataclass(frozen=True)
class SparseAttentionConfig:
    """Block-sparse attention geometry (args.py:135-181)."""

    index_dim: int
    num_index_heads: int
    block_size: int
    topk_blocks: int
    local_blocks: int
    init_blocks: int


@dataclass(frozen=True)
class MiniMaxM3Config:
    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rotary_dim: int
    rope_theta: float
    max_position_embeddings: int
    rms_norm_eps: float
    use_qk_norm: bool
    use_gemma_norm: bool
    tie_word_embeddings: bool
    # feed-forward
    hidden_act: str
    swiglu_alpha: float
    swiglu_limit: float
    num_local_experts: int
    num_experts_per_tok: int
    intermediate_size: int
    dense_intermediate_size: int
    shared_intermediate_size: int
    n_shared_experts: int
    routed_scaling_factor: float
    use_routing_bias: bool
    scoring_func: str
    # per-layer choices
    mixer_types: Tuple[str, ...]
    ffn_types: Tuple[str, ...]
    sparse: Optional[SparseAttentionConfig]
    eos_token_ids: Tuple[int, ...] = ()
    torch_dtype: Optional[str] = None
    wrapped: bool = False  # config.json held the text model under "text_config"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], num_layers: Optional[int] = None) -> "MiniMaxM3Config":
        archs = raw.get("architectures") or [ARCHITECTURES[1]]
        wrapped = isinstance(raw.get("text_config"), Mapping)
        text: Mapping[str, Any] = raw["text_config"] if wrapped else raw

        def need(key: str) -> Any:
            if key not in text or text[key] is None:
                raise ConfigError(f"config.json: required key '{key}' is missing")
            return text[key]

        def integer(key: str, value: Any, minimum: int = 1) -> int:
            if isinstance(value, bool) or not isinstance(value, int) or value < minimum:
                raise ConfigError(f"config.json: '{key}' must be an integer >= {minimum}, got {value!r}")
            return value

        hidden = integer("hidden_size", need("hidden_size"))
        layers_total = integer("num_hidden_layers", need("num_hidden_layers"))
        layers = layers_total
        if num_layers is not None:  # layer cap (config.py:64-76 does this through an env switch)
            if num_layers < 1:
                raise ConfigError(f"num_layers override must be >= 1, got {num_layers}")
            layers = min(layers_total, num_layers)
        heads = integer("num_attention_heads", need("num_attention_heads"))
        kv_heads = integer("num_key_value_heads", text.get("num_key_value_heads") or heads)
        if heads % kv_heads:
            raise ConfigError(
                f"config.json: num_attention_heads={heads} is not a multiple of num_key_value_heads={kv_heads}"
            )
        head_dim = text.get("head_dim") or hidden // heads  # args.py:212-214
        head_dim = integer("head_dim", head_dim)
        rotary_dim = text.get("rotary_dim")
        if rotary_dim is None:  # args.py:215-217
            rotary_dim = int(head_dim * float(text.get("partial_rotary_factor", 1.0)))
        rotary_dim = integer("rotary_dim", rotary_dim, minimum=0)
        if rotary_dim > head_dim or rotary_dim % 2:
            raise ConfigError(
                f"config.json: rotary_dim={rotary_dim} must be even and <= head_dim={head_dim}"
            )

        theta = text.get("rope_theta")
        rope_params = text.get("rope_parameters") or {}
        if theta is None and isinstance(rope_params, Mapping):
            theta = rope_params.get("rope_theta")
        theta = float(theta) if theta is not None else 10000.0  # args.py:91-96
        scaling = text.get("rope_scaling") or rope_params or {}
        rope_type = scaling.get("rope_type", scaling.get("type", "default")) if scaling else "default"
        if rope_type not in (None, "default"):  # args.py:193-198
            raise ConfigError(f"config.json: rope scaling '{rope_type}' is not supported (plain rope only)")

        if bool(text.get("attention_output_gate", False)):  # args.py:204-206
            raise ConfigError("config.json: attention_output_gate=true is not supported")
        if text.get("qk_norm_type", "per_head") != "per_head":  # args.py:207
            raise ConfigError(
                f"config.json: qk_norm_type={text.get('qk_norm_type')!r} is not supported (per_head only)"
            )
        if float(text.get("swiglu_beta", 1.0)) != 1.0:  # args.py:188-189
            raise ConfigError("config.json: swiglu_beta must be 1.0")
        act = text.get("hidden_act", "swigluoai")
        if act not in ("swigluoai", "silu"):  # config.py:132-135
            raise ConfigError(f"config.json: hidden_act={act!r} is not supported (swigluoai or silu)")
        if act == "silu" and ("swiglu_alpha" in text or "swiglu_limit" in text):
            # the native key shape spells the clamped activation "silu" but keeps its constants; the
            # reference runs swigluoai for it (config.py:128-145).  "silu" without them is plain SwiGLU.
            act = "swigluoai"
        scoring = text.get("scoring_func", "sigmoid")
        if scoring not in ("sigmoid", "softmax"):
            raise ConfigError(f"config.json: scoring_func={scoring!r} is not supported (sigmoid or softmax)")

        # ---- per-layer feed-forward choice (args.py:78-81,125-132)
        freq = text.get("moe_layer_freq")
        if freq is None and text.get("mlp_layer_types") is not None:
            freq = [1 if t == "sparse" else 0 for t in text["mlp_layer_types"]]
        experts = int(text.get("num_local_experts", 0) or 0)
        if not freq:
            ffn_types = [FFN_MOE if experts > 0 else FFN_DENSE] * layers
        else:
            if len(freq) < layers:
                raise ConfigError(
                    f"config.json: moe_layer_freq has {len(freq)} entries, model has {layers} layers"
                )
            ffn_types = [FFN_MOE if f else FFN_DENSE for f in freq[:layers]]
        top_k = int(text.get("num_experts_per_tok", 0) or 0)
        if FFN_MOE in ffn_types:
            if experts < 1:
                raise ConfigError("config.json: MoE layers need num_local_experts >= 1")
            if not 1 <= top_k <= experts:
                raise ConfigError(
                    f"config.json: num_experts_per_tok={top_k} must be in [1, num_local_experts={experts}]"
                )
        inter = integer("intermediate_size", need("intermediate_size"))
        dense_inter = int(text.get("dense_intermediate_size", 0) or inter)  # args.py:238-241
        shared_inter = int(text.get("shared_intermediate_size", 0) or inter)  # args.py:242-245

        # ---- per-layer mixer choice (args.py:99-122,135-181)
        sparse_raw = text.get("sparse_attention_config")
        layer_types = text.get("layer_types") or []
        if not sparse_raw and "minimax_m3_sparse" in layer_types:
            sparse_raw = {
                "use_sparse_attention": True,
                "sparse_attention_freq": [1 if t == "minimax_m3_sparse" else 0 for t in layer_types],
                "sparse_num_index_heads": int(text.get("index_n_heads", 4)),
                "sparse_index_dim": int(text.get("index_head_dim", 128)),
                "sparse_block_size": int(text.get("index_block_size", 128)),
                "sparse_topk_blocks": int(text.get("index_topk_blocks", 16)),
                "sparse_local_block": int(text.get("index_local_blocks", 1)),
                "sparse_init_block": 0,
                "sparse_score_type": "max",
            }
        mixer_types = [MIXER_FULL] * layers
        sparse_cfg: Optional[SparseAttentionConfig] = None
        alias = text.get("attn_type_list")
        if alias is not None:
            if len(alias) < layers:
                raise ConfigError(
                    f"config.json: attn_type_list has {len(alias)} entries, model has {layers} layers"
                )
            for i, a in enumerate(alias[:layers]):
                if a not in (0, MIXER_FULL, "full_attention"):
                    raise ConfigError(
                        f"config.json: attn_type_list[{i}]={a!r} names a mixer this engine does not have"
                    )
        if sparse_raw and bool(sparse_raw.get("use_sparse_attention", False)):
            if sparse_raw.get("sparse_score_type", "max") != "max":  # args.py:147-151
                raise ConfigError("config.json: sparse_score_type must be 'max'")
            sfreq = sparse_raw.get("sparse_attention_freq")
            ids = list(range(layers)) if not sfreq else [i for i, f in enumerate(sfreq[:layers]) if f]
            disable_value = sparse_raw.get("sparse_disable_index_value")
            if disable_value is not None and not all(
                bool(disable_value[i]) for i in ids if i < len(disable_value)
            ):  # args.py:154-158
                raise ConfigError("config.json: sparse layers must set sparse_disable_index_value")
            block = int(sparse_raw.get("sparse_block_size", 128))
            if block < 1:
                raise ConfigError("config.json: sparse_block_size must be >= 1")
            index_dim = int(sparse_raw.get("sparse_index_dim", 0))
            if index_dim != head_dim:  # args.py:167-171
                raise ConfigError(
                    f"config.json: sparse_index_dim={index_dim} must equal head_dim={head_dim}"
                )
            topk = int(sparse_raw.get("sparse_topk_blocks", 0))
            if not 0 < topk < 64:  # args.py:172-176
                raise ConfigError(f"config.json: sparse_topk_blocks={topk} must be in (0, 64)")
            local = int(sparse_raw.get("sparse_local_block", 0))
            if local < 1:  # args.py:177-181
                raise ConfigError("config.json: sparse_local_block must be >= 1")
            index_heads = int(sparse_raw.get("sparse_num_index_heads", 0))
            if index_heads != kv_heads:  # args.py:222-225
                raise ConfigError(
                    f"config.json: sparse_num_index_heads={index_heads} must equal num_key_value_heads={kv_heads}"
                )
            if ids:
                sparse_cfg = SparseAttentionConfig(
                    index_dim=index_dim,
                    num_index_heads=index_heads,
                    block_size=block,
                    topk_blocks=topk,
                    local_blocks=local,
                    init_blocks=int(sparse_raw.get("sparse_init_block", 0)),
                )
                for i in ids:
                    mixer_types[i] = MIXER_SPARSE

        eos = text.get("eos_token_id", raw.get("eos_token_id"))
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)

        dtype = text.get("torch_dtype") or text.get("dtype") or raw.get("torch_dtype") or raw.get("dtype")
        return cls(
            architecture=str(archs[0]),
            vocab_size=integer("vocab_size", need("vocab_size")),
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rotary_dim=rotary_dim,
            rope_theta=theta,
            max_position_embeddings=integer(
                "max_position_embeddings", text.get("max_position_embeddings", 4096)
            ),
            rms_norm_eps=float(need("rms_norm_eps")),
            use_qk_norm=bool(text.get("use_qk_norm", True)),
            use_gemma_norm=bool(text.get("use_gemma_norm", True)),
            tie_word_embeddings=bool(
                text.get("tie_word_embeddings", raw.get("tie_word_embeddings", False))
            ),
            hidden_act=act,
            swiglu_alpha=float(text.get("swiglu_alpha", 1.702)),
            swiglu_limit=float(text.get("swiglu_limit", 7.0)),
            num_local_experts=experts,
            num_experts_per_tok=top_k,
            intermediate_size=inter,
            dense_intermediate_size=dense_inter,
            shared_intermediate_size=shared_inter,
            n_shared_experts=int(text.get("n_shared_experts", 0) or 0),
            routed_scaling_factor=float(text.get("routed_scaling_factor", 1.0)),
            use_routing_bias=bool(text.get("use_routing_bias", False)),
            scoring_func=scoring,
            mixer_types=tuple(mixer_types),
            ffn_types=tuple(ffn_types),
            sparse=sparse_cfg,
            eos_token_ids=eos_ids,
            torch_dtype=str(dtype) if dtype is not None else None,
            wrapped=wrapped,
        )

    @classmethod
    def from_folder(cls, folder: str, num_layers: Optional[int] = None) -> "MiniMaxM3Config":
        return cls.from_dict(read_config_json(folder), num_layers=num_layers)

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        """config.json contents (raw checkpoint key shape) that read back to this config."""
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "minimax_m3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rotary_dim": self.rotary_dim,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "use_qk_norm": self.use_qk_norm,
            "qk_norm_type": "per_head",
            "use_gemma_norm": self.use_gemma_norm,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "num_local_experts": self.num_local_experts,
            "num_experts_per_tok": self.num_experts_per_tok,
            "intermediate_size": self.intermediate_size,
            "dense_intermediate_size": self.dense_intermediate_size,
            "shared_intermediate_size": self.shared_intermediate_size,
            "n_shared_experts": self.n_shared_experts,
            "routed_scaling_factor": self.routed_scaling_factor,
            "use_routing_bias": self.use_routing_bias,
            "scoring_func": self.scoring_func,
            "moe_layer_freq": [1 if t == FFN_MOE else 0 for t in self.ffn_types],
            # (only beside the clamped activation: next to "silu" they would turn it into swigluoai)
            **({"swiglu_alpha": self.swiglu_alpha, "swiglu_limit": self.swiglu_limit}
               if self.hidden_act == "swigluoai" else {}),
            "torch_dtype": self.torch_dtype or "bfloat16",
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.sparse is not None:
            out["sparse_attention_config"] = {
                "use_sparse_attention": True,
                "sparse_attention_freq": [1 if t == MIXER_SPARSE else 0 for t in self.mixer_types],
                "sparse_num_index_heads": self.sparse.num_index_heads,
                "sparse_index_dim": self.sparse.index_dim,
                "sparse_block_size": self.sparse.block_size,
                "sparse_topk_blocks": self.sparse.topk_blocks,
                "sparse_local_block": self.sparse.local_blocks,
                "sparse_init_block": self.sparse.init_blocks,
                "sparse_score_type": "max",
                "sparse_disable_index_value": [1] * self.num_hidden_layers,
            }
        return out

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads
