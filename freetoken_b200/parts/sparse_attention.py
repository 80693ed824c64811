"""Block-sparse grouped-query attention (the layers a config flags as sparse).

On top of the dense mixer (python/freetoken/models/minimax_m3/attention.py:94-112): an index
projection gives one index query per KV head and one shared index key per token, both normed
and rotated like q and k (:95-104); index keys are cached for every token
(python/freetoken/attention/m3_sparse.py:256-259).  A block's score is the largest
``index_q . index_k`` over its visible positions, unscaled
(python/freetoken/kernel/triton/minimax_m3_sparse.py:152-170); the first ``init_blocks`` and the
newest ``local_blocks`` blocks are always taken, then the best of the rest up to ``topk_blocks``
(:232-284); each KV head's query group attends only the keys of its chosen blocks (:601-684).
While a sequence is no longer than ``topk_blocks * block_size`` this equals dense attention.
"""

from __future__ import annotations

from typing import Any, Dict

import torch

from ..config.spec import PagedKVNeed, ParamSpec, PartSpec
from ..errors import ConfigError
from ..kernels import ops
from .attention import GQAttention
from .base import MIXERS, BuildEnv, StepState


@MIXERS.register("block_sparse_attention")
class BlockSparseAttention(GQAttention):
    """params: those of ``gqa_attention`` plus ``index_dim``, ``n_index_heads``, ``block_size``,
    ``topk_blocks``, ``local_blocks``, ``init_blocks``."""

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.index_dim = int(spec["index_dim"])
        self.n_index_heads = int(spec["n_index_heads"])
        self.block_size = int(spec["block_size"])
        self.topk_blocks = int(spec["topk_blocks"])
        self.local_blocks = int(spec["local_blocks"])
        self.init_blocks = int(spec.get("init_blocks", 0))
        if self.n_index_heads != self.n_kv_heads:
            raise ConfigError("block_sparse_attention: one index head per KV head is required")
        if self.index_dim != self.head_dim:
            raise ConfigError("block_sparse_attention: index_dim must equal head_dim (shared rotation)")
        if self.window is not None:
            raise ConfigError("block_sparse_attention: a window cannot be combined with block selection")

    def param_specs(self) -> Dict[str, ParamSpec]:
        out = super().param_specs()
        out["index_qk_proj.weight"] = ParamSpec(((self.n_index_heads + 1) * self.index_dim, self.hidden))
        init = ("normal", 0.0, 0.02) if self.gemma else ("normal", 1.0, 0.02)
        out["index_q_norm.weight"] = ParamSpec((self.index_dim,), "float32", init, store="bfloat16")
        out["index_k_norm.weight"] = ParamSpec((self.index_dim,), "float32", init, store="bfloat16")
        return out

    def cache_need(self):
        return PagedKVNeed((("k", self.n_kv_heads, self.head_dim), ("v", self.n_kv_heads, self.head_dim),
                            ("index_k", 1, self.index_dim)), None)

    def plan_key(self, decode_only: bool = False):
        return ("sparse_attention", self.group, self.n_kv_heads, self.head_dim, self.block_size, self.topk_blocks)

    def prepare(self, builder) -> None:
        builder.sparse_attention_plan(self)

    def forward(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        return sparse_forward(self, h, step, cache, writes_cache)


def sparse_forward(m: BlockSparseAttention, h, step, cache, writes_cache):
    from ..errors import KernelError

    raise KernelError("block_sparse_attention: the block-selection kernels are not built yet")
