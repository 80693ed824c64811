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
        if self.group > 16:
            raise ConfigError(f"block_sparse_attention: {self.group} query heads per KV head exceed the "
                              f"kernel's 16-row tile")

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

    graph_safe = True

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        index = n_tokens * ((2 * self.n_index_heads + 1) * self.index_dim * item + self.n_kv_heads * self.topk_blocks * 4
                            + self.n_index_heads * -(-self.env.max_seq_len // self.block_size) * 4)  # (+ block scores)
        return super().workspace_bytes(n_tokens) + index

    def plan_key(self, decode_only: bool = False):
        return ("sparse_attention", self.group, 16, self.n_kv_heads, self.head_dim, self.block_size,
                self.topk_blocks)

    def prepare(self, builder) -> None:
        # the longest request's length rounded up to a power of two: what a step replayed from a graph may
        # depend on (the engine records a new graph when it changes)
        self._span = builder.longest_span()
        builder.sparse_attention_plan(self.group, 16, self.n_kv_heads, self.head_dim, self.block_size,
                                      self.topk_blocks)

    def forward(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        Hq, Hkv, D, Hi = self.n_heads, self.n_kv_heads, self.head_dim, self.n_index_heads
        # main projection, norm, rotation, cache write: as in the dense mixer
        n_proj = self.q_dim + (2 * self.kv_dim if writes_cache else 0)
        qkv = ws.get("attn.qkv", (T, n_proj), dt, (cap, self.q_dim + 2 * self.kv_dim))
        w = self.params["qkv_proj.weight"]
        ops.linear(h, w if writes_cache else w[: self.q_dim], qkv)
        q = ws.get("attn.q", (T, Hq, D), dt, (cap, Hq, D))
        sections = [dict(first_head=0, n_heads=Hq, norm_weight=self.params.get("q_norm.weight"), rotate=True,
                         dense_out=q)]
        if writes_cache:
            sections.append(dict(first_head=Hq, n_heads=Hkv, norm_weight=self.params.get("k_norm.weight"),
                                 rotate=True, slab=cache.slabs["k"], slot_map=cache.slot_map))
            sections.append(dict(first_head=Hq + Hkv, n_heads=Hkv, norm_weight=None, rotate=False,
                                 slab=cache.slabs["v"], slot_map=cache.slot_map))
        ops.norm_rope_store(qkv, D, self.rotary_dim, step.positions, self.position.table(), self.eps,
                            self.gemma, sections)
        # index queries (one per KV head) and the shared index key, normed and rotated the same way
        n_index = (Hi + (1 if writes_cache else 0)) * self.index_dim
        iqk = ws.get("attn.iqk", (T, n_index), dt, (cap, (Hi + 1) * self.index_dim))
        wi = self.params["index_qk_proj.weight"]
        ops.linear(h, wi if writes_cache else wi[: Hi * self.index_dim], iqk)
        iq = ws.get("attn.iq", (T, Hi, self.index_dim), dt, (cap, Hi, self.index_dim))
        sections = [dict(first_head=0, n_heads=Hi, norm_weight=self.params["index_q_norm.weight"], rotate=True,
                         dense_out=iq)]
        if writes_cache:
            sections.append(dict(first_head=Hi, n_heads=1, norm_weight=self.params["index_k_norm.weight"],
                                 rotate=True, slab=cache.slabs["index_k"], slot_map=cache.slot_map))
        ops.norm_rope_store(iqk, self.index_dim, self.rotary_dim, step.positions, self.position.table(),
                            self.eps, self.gemma, sections)
        # which key blocks each token reads, then attention over those
        sel = ws.get("attn.sel", (T, Hkv, self.topk_blocks), torch.int32, (cap, Hkv, self.topk_blocks))
        max_blocks = -(-self.env.max_seq_len // self.block_size)
        scores = None
        if dt == torch.bfloat16 and ops.sparse_score_fits(Hi, self.index_dim, self.block_size):
            scores = ws.get("attn.block_scores", (T, Hi, max_blocks), torch.float32, (cap, Hi, max_blocks))
        ops.sparse_select(iq, cache.slabs["index_k"], cache.block_table, step.seg_info, len(step.segments),
                          self.block_size, self.local_blocks, self.init_blocks, max_blocks, sel, scores,
                          live_blocks=min(max_blocks, -(-self._span // self.block_size)))
        plan = step.attention_plans[self.plan_key()]
        o = ws.get("attn.o", (T, Hq, D), dt, (cap, Hq, D))
        ops.paged_attention(q, cache.slabs["k"], cache.slabs["v"], cache.block_table, step.seg_info,
                            len(step.segments), plan.items_dev, plan.n_items, plan.part_o, plan.part_ml, o, 16,
                            self.scale, None, sel=sel, block_size=self.block_size)
        out = ws.get("attn.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(o.view(T, self.q_dim), self.params["o_proj.weight"], out)
        return out
