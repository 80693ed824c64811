"""Packing one step's metadata into a single host-to-device copy.

Everything the kernels need to know about a step is int32: token ids, positions, cache
slots of the new tokens per paged group, per-segment (q_start, q_len, kv_len, block-table
row), state slots, the rows whose logits are wanted, block-table changes, and the attention
work lists.  The sections are laid out back to back (16-byte aligned) in one pinned host
buffer and copied once; kernels read them through views of the device buffer.  The
reference stages the same quantities as several pinned tensors
(python/freetoken/scheduler/scheduler.py:874-905, python/freetoken/attention/triton.py:229-240).

A step whose layout is *fixed* (decode-only steps replayed from a CUDA graph) pads its
variable sections to a size that depends only on the batch size, so that every replay
finds each section at the same address.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .attention_plan import TC_ONE_TILE_COSTS, TC_TWO_TILE_COSTS, AttentionPlan, build_plan, wave_splits

ALIGN = 4  # int32 elements = 16 bytes


@dataclass
class DevicePlan:
    """An attention work list on the device, with its scratch for split tiles."""

    items_dev: torch.Tensor
    n_items: int
    part_o: Optional[torch.Tensor]
    part_ml: Optional[torch.Tensor]
    host: AttentionPlan


class StepBuffers:
    """Pinned staging (double-buffered) and the device copy of the packed metadata."""

    def __init__(self, device: torch.device, capacity_ints: int):
        self.device = device
        self.capacity = capacity_ints
        pin = device.type == "cuda"
        self.host = [torch.empty(capacity_ints, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.host_np = [h.numpy() for h in self.host]
        self.dev = torch.zeros(capacity_ints, dtype=torch.int32, device=device)
        self.events: List[Optional[Any]] = [None, None]
        self.turn = 0
        self.last_upload_bytes = 0

    def grow(self, need: int) -> None:
        if need <= self.capacity:
            return
        raise RuntimeError(
            f"step metadata needs {need} int32, the buffer holds {self.capacity}; "
            f"raise max_step_tokens / max_running_req")

    def upload(self, sections: List[Tuple[str, np.ndarray]]) -> Dict[str, torch.Tensor]:
        offsets = []
        n = 0
        for _, arr in sections:
            offsets.append(n)
            n += -(-max(arr.size, 1) // ALIGN) * ALIGN
        self.grow(n)
        i = self.turn
        self.turn ^= 1
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.host_np[i]
        for (name, arr), off in zip(sections, offsets):
            buf[off:off + arr.size] = arr.reshape(-1)
        self.last_upload_bytes = 4 * n
        if n:
            self.dev[:n].copy_(self.host[i][:n], non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self.events[i] = ev
        out = {}
        for (name, arr), off in zip(sections, offsets):
            out[name] = self.dev[off:off + arr.size].view(arr.shape)
        return out


class StepBuilder:
    """Collects the sections of one step; mixers add what their kernels need."""

    def __init__(self, engine, seg_lens: Sequence[Tuple[int, int]], fixed: bool, sm_count: int):
        self.engine = engine
        self.seg_lens = list(seg_lens)  # (q_len, kv_len) per segment
        self.fixed = fixed
        self.sm_count = sm_count
        self.sections: List[Tuple[str, np.ndarray]] = []
        self.decode_only = all(q == 1 for q, _ in self.seg_lens)
        self.plans: Dict[Any, AttentionPlan] = {}
        self._drafts: Dict[Any, AttentionPlan] = {}  # work lists made to compare kernel forms, not (yet) part of the step
        self.plan_dims: Dict[Any, Tuple[int, int, int]] = {}

    def add(self, name: str, arr: np.ndarray) -> None:
        self.sections.append((name, np.ascontiguousarray(arr, dtype=np.int32)))

    def longest_span(self) -> int:
        """The longest request's length rounded up to a power of two: what a graph-replayed decode
        step may let its kernel choice and split count depend on (it changes a handful of times as
        requests grow)."""
        longest = max(kv for _, kv in self.seg_lens)
        return 1 << max(6, (longest - 1).bit_length())

    def fixed_splits(self, n_kv_heads: int, ctas_per_sm: int = 2) -> int:
        """Splits per tile of a graph-replayed decode step: enough CTAs to fill the GPU at
        this batch size, independent of the requests' exact lengths."""
        b = max(1, len(self.seg_lens))
        return wave_splits(b * n_kv_heads, ctas_per_sm * self.sm_count, 16, self.longest_span())

    def attention_plan(self, group: int, tile_rows: int, window: Optional[int], n_kv_heads: int,
                       head_dim: int, few_rows: bool = False) -> Any:
        """``few_rows``: the work list is for the tcgen05 kernel in its form for tiles of at most 16 rows (key tiles of 128)."""
        key = ("attention", group, tile_rows, window, n_kv_heads, head_dim, few_rows)
        if key not in self.plans:
            plan = self._drafts.pop(key, None) or self._draft(group, tile_rows, window, n_kv_heads, few_rows)
            self.plans[key] = plan
            self.plan_dims[key] = (n_kv_heads, tile_rows, head_dim)
            self.add(f"plan.{len(self.plans) - 1}", plan.items)
        return key

    def _draft(self, group: int, tile_rows: int, window: Optional[int], n_kv_heads: int, few_rows: bool) -> AttentionPlan:
        tensor_core = tile_rows >= 128 or few_rows
        per_sm = 1 if tensor_core else 2  # the tcgen05 kernels fill an SM with one CTA
        costs = None
        if tile_rows >= 128 and not self.fixed:  # what a piece costs these kernels: for the cuts and for est_us
            costs = TC_TWO_TILE_COSTS if tile_rows == 256 else TC_ONE_TILE_COSTS
        return build_plan(self.seg_lens, group, tile_rows, window, n_kv_heads,
                          sm_count=self.sm_count if per_sm == 2 else max(1, self.sm_count // 2),
                          fixed_splits=self.fixed_splits(n_kv_heads, per_sm) if self.fixed else None,
                          key_tile=128 if tensor_core else 0, costs=costs)

    def cheaper_attention_rows(self, group: int, window: Optional[int], n_kv_heads: int, head_dim: int) -> int:
        """128 or 256: the tcgen05 attention kernel (one or two query tiles a piece) whose work list for this step
        is estimated to end sooner; the two-tile form has to be ahead by 3 %.  The list of the form chosen is
        kept for :meth:`attention_plan`."""
        est = {}
        for rows in (128, 256):
            key = ("attention", group, rows, window, n_kv_heads, head_dim, False)
            plan = self.plans.get(key) or self._drafts.get(key)
            if plan is None:
                plan = self._drafts[key] = self._draft(group, rows, window, n_kv_heads, False)
            est[rows] = plan.est_us
        if est[128] is None or est[256] is None:
            return 128
        return 256 if est[256] < 0.97 * est[128] else 128

    def sparse_attention_plan(self, group: int, tile_rows: int, n_kv_heads: int, head_dim: int,
                              block_size: int, topk: int) -> Any:
        """Work list of a block-sparse layer: one token per tile, key ranges over chosen keys."""
        key = ("sparse_attention", group, tile_rows, n_kv_heads, head_dim, block_size, topk)
        if key not in self.plans:
            plan = build_plan(self.seg_lens, group, tile_rows, None, n_kv_heads, sm_count=self.sm_count,
                              fixed_splits=self.fixed_splits(n_kv_heads) if self.fixed else None,
                              sparse=(block_size, topk))
            self.plans[key] = plan
            self.plan_dims[key] = (n_kv_heads, tile_rows, head_dim)
            self.add(f"plan.{len(self.plans) - 1}", plan.items)
        return key

    def finish(self, buffers: StepBuffers, workspace) -> Tuple[Dict[str, torch.Tensor], Dict[Any, DevicePlan]]:
        tensors = buffers.upload(self.sections)
        plans: Dict[Any, DevicePlan] = {}
        for i, (key, plan) in enumerate(self.plans.items()):
            n_kv, rows, dim = self.plan_dims[key]
            part_o = part_ml = None
            if plan.n_slots:
                tag = f"attn.part.{i}.fixed{len(self.seg_lens)}x{plan.n_slots}x{rows}" if self.fixed else f"attn.part.{i}"
                part_o = workspace.get(tag + ".o", (plan.n_slots, n_kv, rows, dim), torch.float32)
                part_ml = workspace.get(tag + ".ml", (plan.n_slots, n_kv, rows, 2), torch.float32)
            plans[key] = DevicePlan(tensors[f"plan.{i}"], plan.n_items, part_o, part_ml, plan)
        return tensors, plans
