"""Grouped-query softmax attention over a paged cache.

Order of operations (python/freetoken/models/minimax_m3/attention.py:79-119): fused qkv
projection (rows q, k, v), per-head RMSNorm of q and k heads with one ``[head_dim]`` weight
each (:54-56,90-91), partial NeoX rotation of q and k (:92), keys and values of the new
tokens stored in the cache before it is read (python/freetoken/attention/triton.py:150),
causal softmax attention with scale ``head_dim^-0.5`` where query head ``h`` reads KV head
``h // group`` (python/freetoken/kernel/triton/attention.py:74,102,118-137), output
projection.  Norm, rotation and the page write are one kernel here; the projections are
library matrix products, as in the reference (python/freetoken/layers/linear.py:31-32).
"""

from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch

from ..config.spec import PagedKVNeed, ParamSpec, PartSpec
from ..engine.attention_plan import DEAL_MOST_PIECES
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, BuildEnv, Mixer, StepState
from .rope import shared_position


TC_MIN_TOKENS = 128      # shortest step that goes to the tcgen05 attention kernel
TC_PAIR_MIN_TOKENS = 1024  # from this many tokens on, a step goes to the kernel with two query tiles per CTA
TC_PAIR_MIN_TOKENS_LONG = 256  # ... and from this many on when its longest request has TC_PAIR_MIN_SPAN keys and more
TC_PAIR_MIN_SPAN = 16384       # (rounded up to 2^n): such tiles are cut along the keys into enough pieces for every SM
TC_MIN_DECODE_SPAN = 0   # decode steps go there from this length of the longest request (rounded up to 2^n) on


def attention_kernel_form(dtype: torch.dtype, decode_only: bool = False, group: int = 1, n_tokens: int = 0,
                          head_dim: int = 0, page_size: int = 0, window: Optional[int] = None,
                          longest_span: int = 0) -> Tuple[int, bool]:
    """``(query rows one attention CTA handles, the tcgen05 kernel's form for few rows)``.

    16 rows in the 32-bit kernel.  bfloat16 steps whose sizes the tcgen05 kernels take: 128 rows for
    long steps (``TC_MIN_TOKENS`` tokens and more; 256, two such tiles per CTA, from
    ``TC_PAIR_MIN_TOKENS`` tokens on, or from ``TC_PAIR_MIN_TOKENS_LONG`` for portions of long prompts: the
    rule for callers without a step's work lists; a step itself takes, from ``TC_PAIR_MIN_TOKENS_LONG`` tokens
    on, the form whose work list is estimated to end sooner, see ``GQAttention.prepare``);
    decode steps go to the same kernel in its form for tiles of at
    most 16 rows, where one warp takes the softmax (groups of up to 16 heads; ``longest_span`` is the longest
    request's length rounded up to a power of two, from which on they go there:
    ``TC_MIN_DECODE_SPAN``), larger groups to the 128-row kernel.  Otherwise 16 rows for decode steps
    of small groups and 64 in the bfloat16 mma.sync kernels."""
    if dtype != torch.bfloat16:
        return 16, False
    sized = bool(window is None and head_dim and page_size)
    if decode_only:
        if sized and longest_span >= TC_MIN_DECODE_SPAN:
            if ops.attention_tc_few_fits(head_dim, page_size, group):
                return 16, True
            if ops.attention_tc_fits(head_dim, page_size, group):
                return 128, False
        return (16 if group <= 16 else 64), False
    tc = sized and ops.attention_tc_fits(head_dim, page_size, group)
    if tc and (n_tokens >= TC_PAIR_MIN_TOKENS or
               (n_tokens >= TC_PAIR_MIN_TOKENS_LONG and longest_span >= TC_PAIR_MIN_SPAN)):
        return 256, False
    if tc and n_tokens >= TC_MIN_TOKENS:
        return 128, False
    return 64, False


def attention_tile_rows(dtype: torch.dtype, decode_only: bool = False, group: int = 1, n_tokens: int = 0,
                        head_dim: int = 0, page_size: int = 0, window: Optional[int] = None,
                        longest_span: int = 0) -> int:
    """Query rows (tokens x group heads) one attention CTA handles (see :func:`attention_kernel_form`)."""
    return attention_kernel_form(dtype, decode_only, group, n_tokens, head_dim, page_size, window, longest_span)[0]


@MIXERS.register("gqa_attention")
class GQAttention(Mixer):
    """params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``, ``qk_norm`` (bool),
    ``eps``, ``gemma`` (bool), ``position`` (PartSpec of a position encoding), ``window``
    (None or tokens), ``scale`` (None = head_dim^-0.5)."""

    graph_safe = True  # running a step twice writes the same keys and values again

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden"])
        self.n_heads = int(spec["n_heads"])
        self.n_kv_heads = int(spec["n_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        if self.n_heads % self.n_kv_heads:
            raise ConfigError("gqa_attention: n_heads must be a multiple of n_kv_heads")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ConfigError(
                f"gqa_attention: head_dim={self.head_dim} must be a multiple of 16 in [16, 256]")
        self.group = self.n_heads // self.n_kv_heads
        self.qk_norm = bool(spec.get("qk_norm", True))
        self.eps = float(spec.get("eps", 1e-6))
        self.gemma = bool(spec.get("gemma", True))
        self.window: Optional[int] = spec.get("window")
        self.scale = float(spec.get("scale") or self.head_dim ** -0.5)
        self.position = shared_position(spec.get("position") or PartSpec("none"), env)
        self.rotary_dim = int(getattr(self.position, "rotary_dim", 0))
        if self.rotary_dim > self.head_dim:
            raise ConfigError("gqa_attention: rotary_dim exceeds head_dim")
        if self.group > attention_tile_rows(env.dtype):
            raise ConfigError(
                f"gqa_attention: {self.group} query heads per KV head exceed the kernel's "
                f"{attention_tile_rows(env.dtype)}-row tile")
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv_heads * self.head_dim

    # ------------------------------------------------------------------ tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        out = {
            "qkv_proj.weight": ParamSpec((self.q_dim + 2 * self.kv_dim, self.hidden)),
            "o_proj.weight": ParamSpec((self.hidden, self.q_dim)),
        }
        if self.qk_norm:
            init = ("normal", 0.0, 0.02) if self.gemma else ("normal", 1.0, 0.02)
            out["q_norm.weight"] = ParamSpec((self.head_dim,), "float32", init, store="bfloat16")
            out["k_norm.weight"] = ParamSpec((self.head_dim,), "float32", init, store="bfloat16")
        return out

    def cache_need(self):
        return PagedKVNeed((("k", self.n_kv_heads, self.head_dim),
                            ("v", self.n_kv_heads, self.head_dim)), self.window)

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        # qkv, q, o, out; and the 32-bit partial results of tiles split along the keys (at most
        # attention_plan.DEAL_MOST_PIECES pieces per SM, 256 rows each at most)
        rows = n_tokens * (3 * self.q_dim + 2 * self.kv_dim + self.hidden) * item
        return rows + DEAL_MOST_PIECES * 148 * 256 * (self.head_dim + 2) * 4

    # ------------------------------------------------------------------ step
    def kernel_form(self, decode_only: bool, n_tokens: int = 0, page_size: int = 0, longest_span: int = 0):
        return attention_kernel_form(self.env.dtype, decode_only, self.group, n_tokens, self.head_dim, page_size,
                                     self.window, longest_span)

    def tile_rows(self, decode_only: bool, n_tokens: int = 0, page_size: int = 0, longest_span: int = 0) -> int:
        return self.kernel_form(decode_only, n_tokens, page_size, longest_span)[0]

    def plan_key(self, decode_only: bool = False, n_tokens: int = 0, page_size: int = 0, longest_span: int = 0):
        rows, few_rows = self.kernel_form(decode_only, n_tokens, page_size, longest_span)
        return ("attention", self.group, rows, self.window, self.n_kv_heads, self.head_dim, few_rows)

    def prepare(self, builder) -> None:
        """Ask the step for the work list this mixer's attention kernel runs from."""
        n_tokens = sum(q for q, _ in builder.seg_lens)
        page_size = builder.engine.config.page_size if builder.engine is not None else 0
        # forward() of the same step runs the kernel this work list was made for
        rows, few_rows = self.kernel_form(builder.decode_only, n_tokens, page_size, builder.longest_span())
        if rows >= 128 and not few_rows and not builder.decode_only and n_tokens >= TC_PAIR_MIN_TOKENS_LONG \
                and hasattr(builder, "cheaper_attention_rows"):
            # one or two query tiles a piece: whichever work list the kernel is estimated to get through sooner
            rows = builder.cheaper_attention_rows(self.group, self.window, self.n_kv_heads, self.head_dim)
        self._step_plan = builder.attention_plan(self.group, rows, self.window, self.n_kv_heads, self.head_dim,
                                                 few_rows)

    def forward(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        T = h.shape[0]
        ws, dt = self.env.workspace, self.env.dtype
        cap = self.env.max_step_tokens
        n_proj = self.q_dim + (2 * self.kv_dim if writes_cache else 0)
        qkv = ws.get("attn.qkv", (T, n_proj), dt, (cap, self.q_dim + 2 * self.kv_dim))
        w = self.params["qkv_proj.weight"]
        ops.linear(h, w if writes_cache else w[: self.q_dim], qkv)
        q = ws.get("attn.q", (T, self.n_heads, self.head_dim), dt, (cap, self.n_heads, self.head_dim))
        sections = [dict(first_head=0, n_heads=self.n_heads,
                         norm_weight=self.params.get("q_norm.weight"), rotate=True, dense_out=q)]
        if writes_cache:
            sections.append(dict(first_head=self.n_heads, n_heads=self.n_kv_heads,
                                 norm_weight=self.params.get("k_norm.weight"), rotate=True,
                                 slab=cache.slabs["k"], slot_map=cache.slot_map))
            sections.append(dict(first_head=self.n_heads + self.n_kv_heads, n_heads=self.n_kv_heads,
                                 norm_weight=None, rotate=False,
                                 slab=cache.slabs["v"], slot_map=cache.slot_map))
        ops.norm_rope_store(qkv, self.head_dim, self.rotary_dim, step.positions,
                            self.position.table(), self.eps, self.gemma, sections)
        plan = step.attention_plans[self._step_plan]
        o = ws.get("attn.o", (T, self.n_heads, self.head_dim), dt, (cap, self.n_heads, self.head_dim))
        ops.paged_attention(q, cache.slabs["k"], cache.slabs["v"], cache.block_table, step.seg_info,
                            len(step.segments), plan.items_dev, plan.n_items, plan.part_o, plan.part_ml,
                            o, self._step_plan[2], self.scale, self.window, few_rows=self._step_plan[6])
        out = ws.get("attn.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(o.view(T, self.q_dim), self.params["o_proj.weight"], out)
        return out
