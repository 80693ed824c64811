"""The cache manager: who holds which page and which state slot.

Schedule entries whose mixers declare equal needs form a *group*.  A paged group
(:class:`PagedGroup`) owns one page pool, one slab per stored quantity and entry, and one
block table; a group whose need has a ``window`` gives pages back as soon as every position
in them is older than any query can still read.  Groups with different needs have pools of
their own, so a windowed group never competes with a full one.  State groups
(:class:`StateGroup`) hold one fixed-size slot per live request.

The manager is host-side bookkeeping plus the device tensors; block-table changes are
queued as (flat index, page) pairs that the engine ships with the step's metadata.  The
reference spreads the same duties over ``CacheManager`` / ``TableManager``
(python/freetoken/scheduler/cache.py:32-63,256-332,533-571, python/freetoken/scheduler/table.py:4-30),
the pools (python/freetoken/kvcache/mha_pool.py:12-148) and the group specs
(python/freetoken/models/config.py:87-111); it has no prefix reuse here (its ``naive`` cache,
python/freetoken/kvcache/naive_cache.py:16-45): everything a request holds returns to the free
lists when it ends.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..config.spec import PagedKVNeed, StateNeed
from ..errors import CacheError
from .pages import NULL_PAGE, PagePool
from .state import StateSlotPool

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class PagedCacheView:
    """What a mixer sees of its paged cache during one step."""

    slabs: Dict[str, torch.Tensor]  # name -> [pages, heads, page_size, dim] of this entry
    block_table: torch.Tensor  # [max_requests, width] int32, device
    slot_map: Optional[torch.Tensor]  # [T] int32 slot of each new token (set per step)
    page_size: int
    window: Optional[int]
    group: "PagedGroup"


@dataclass
class StateCacheView:
    """What a mixer sees of its per-request state: ``tensors[name][slot]``."""

    tensors: Dict[str, torch.Tensor]  # name -> [num_slots + 1, *shape] of this entry
    group: "StateGroup"


class PagedGroup:
    def __init__(self, index: int, need: PagedKVNeed, entries: List[int], page_size: int,
                 num_pages: int, max_requests: int, width: int, dtype: torch.dtype,
                 device: torch.device, poison: bool):
        self.index = index
        self.need = need
        self.entries = entries
        self.page_size = page_size
        self.width = width
        self.pool = PagePool(num_pages)
        self.slabs: Dict[str, torch.Tensor] = {}
        for name, heads, dim in need.slabs:
            shape = (len(entries), num_pages + 1, heads, page_size, dim)
            t = torch.empty(shape, dtype=dtype, device=device)
            if poison:
                t.fill_(float("nan"))
            else:
                t[:, NULL_PAGE].zero_()
            self.slabs[name] = t
        self.table_host = np.zeros((max_requests, width), dtype=np.int32)
        self.table_dev = torch.zeros((max_requests, width), dtype=torch.int32, device=device)
        self.updates: List[Tuple[int, int]] = []  # (flat index into the table, page)
        self.first_live: Dict[int, int] = {}  # row -> first logical block still held

    def bytes_per_page(self, itemsize: int) -> int:
        return sum(h * d for _, h, d in self.need.slabs) * self.page_size * itemsize * len(self.entries)

    def set_entry(self, row: int, block: int, page: int) -> None:
        """Record a block-table entry.  Only entries that gain a page travel to the device:
        an entry whose page was given back is never read again (it lies beyond the request's
        length or before its window) until a later allocation overwrites it."""
        self.table_host[row, block] = page
        if page != NULL_PAGE:
            self.updates.append((row * self.width + block, page))

    def held_pages(self, row: int, n_blocks: int) -> List[int]:
        return [int(p) for p in self.table_host[row, :n_blocks] if p != NULL_PAGE]

    def dead_blocks(self, length: int) -> int:
        """Logical blocks no later query can read once the request holds ``length`` tokens."""
        if self.need.window is None:
            return 0
        # the next query sits at position `length` and reads positions > length - window
        first_needed = max(0, length - self.need.window + 1)
        return first_needed // self.page_size


class StateGroup:
    def __init__(self, index: int, need: StateNeed, entries: List[int], num_slots: int,
                 device: torch.device):
        self.index = index
        self.need = need
        self.entries = entries
        self.tensors: Dict[str, torch.Tensor] = {}
        for name, shape, dtype in need.tensors:
            self.tensors[name] = torch.zeros((len(entries), num_slots + 1, *shape),
                                             dtype=_DTYPES[dtype], device=device)


@dataclass
class _Request:
    row: int
    length: int = 0
    state_slot: int = 0
    reserved: int = 0  # tokens of the step in flight (pages taken, length not yet advanced)


@dataclass
class StepCachePlan:
    """Result of :meth:`CacheManager.begin_step` (host side)."""

    rows: List[int]
    kv_lens: List[int]
    state_slots: List[int]
    fresh: List[bool]
    slot_maps: List[np.ndarray]  # per paged group: [T] int32


class CacheManager:
    def __init__(self, needs: Sequence[Tuple[int, Any]], page_size: int, num_pages: int,
                 max_requests: int, max_seq_len: int, dtype: torch.dtype, device: torch.device,
                 poison: bool = False, max_step_tokens: Optional[int] = None):
        """``needs``: (schedule entry index, ``PagedKVNeed`` | ``StateNeed``) for every entry
        that owns a cache.  ``num_pages`` usable pages per full paged group; a windowed group
        gets what its window can ever hold."""
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_seq_len = max_seq_len
        self.width = -(-max_seq_len // page_size)
        self.device = device
        self.paged: List[PagedGroup] = []
        self.state: List[StateGroup] = []
        self._entry_group: Dict[int, Tuple[str, int, int]] = {}  # entry -> (kind, group, local)
        by_key: Dict[Hashable, List[int]] = {}
        need_of: Dict[Hashable, Any] = {}
        for entry, need in needs:
            if need is None:
                continue
            if not isinstance(need, (PagedKVNeed, StateNeed)):
                raise CacheError(f"entry {entry}: unknown cache need {need!r}")
            by_key.setdefault(need.group_key(), []).append(entry)
            need_of[need.group_key()] = need
        step = max_step_tokens or max_seq_len
        self.max_step_tokens = step
        for key, entries in by_key.items():
            need = need_of[key]
            if isinstance(need, PagedKVNeed):
                n = num_pages
                if need.window is not None:
                    per_req = -(-(need.window + step) // page_size) + 1
                    n = min(num_pages, max_requests * per_req)
                g = PagedGroup(len(self.paged), need, entries, page_size, n, max_requests,
                               self.width, dtype, device, poison)
                self.paged.append(g)
                for local, e in enumerate(entries):
                    self._entry_group[e] = ("paged", g.index, local)
            else:
                g = StateGroup(len(self.state), need, entries, max_requests, device)
                self.state.append(g)
                for local, e in enumerate(entries):
                    self._entry_group[e] = ("state", g.index, local)
        self.slots = StateSlotPool(max_requests)
        self._rows: List[int] = list(range(max_requests - 1, -1, -1))
        self.requests: Dict[Hashable, _Request] = {}
        self._in_step: List[Tuple[Hashable, int]] = []

    # ------------------------------------------------------------------ sizing
    @staticmethod
    def bytes_per_token(needs: Sequence[Tuple[int, Any]], itemsize: int) -> int:
        """Bytes one cached token costs across all paged entries
        (python/freetoken/kvcache/base.py:19-32 computes the same for its pools)."""
        total = 0
        for _, need in needs:
            if isinstance(need, PagedKVNeed):
                total += sum(h * d for _, h, d in need.slabs) * itemsize
        return total

    # ------------------------------------------------------------------ views
    def view(self, entry: int) -> Any:
        if entry not in self._entry_group:
            return None
        kind, gi, local = self._entry_group[entry]
        if kind == "paged":
            g = self.paged[gi]
            return PagedCacheView({n: t[local] for n, t in g.slabs.items()}, g.table_dev, None,
                                  g.page_size, g.need.window, g)
        g = self.state[gi]
        return StateCacheView({n: t[local] for n, t in g.tensors.items()}, g)

    # ------------------------------------------------------------------ requests
    def open(self, rid: Hashable) -> None:
        if rid in self.requests:
            raise CacheError(f"request {rid!r} is already open")
        if not self._rows:
            raise CacheError(f"no request slot free ({self.max_requests} live requests)")
        row = self._rows.pop()
        self.requests[rid] = _Request(row=row, state_slot=self.slots.alloc())
        for g in self.paged:
            g.first_live[row] = 0

    def is_open(self, rid: Hashable) -> bool:
        return rid in self.requests

    def length(self, rid: Hashable) -> int:
        return self.requests[rid].length

    def free_request_slots(self) -> int:
        return len(self._rows)

    def free_pages(self) -> List[int]:
        return [g.pool.free_count for g in self.paged]

    def pages_for(self, length: int, new_tokens: int, group: PagedGroup, first_live: int = 0) -> int:
        """Pages a request of ``length`` tokens must newly take to hold ``new_tokens`` more."""
        have = -(-length // self.page_size)
        want = -(-(length + new_tokens) // self.page_size)
        return max(0, want - max(have, first_live))

    def pages_to_admit(self, total_tokens: int, step_tokens: Optional[int] = None) -> List[int]:
        """Pages per paged group that a request reaching ``total_tokens`` holds at its peak.

        ``step_tokens``: the most tokens of the request one step carries (default: the engine's
        step size).  A windowed group holds, while a step of ``n`` tokens runs on top of ``L``
        cached ones, the blocks from the first one a query of the step before could still read,
        ``(L - window + 1) // P``, to the last one the step writes, ``ceil((L + n) / P)``: at most
        ``ceil((window - 1 + n) / P) + 1`` pages, whatever ``L`` is."""
        P = self.page_size
        n_step = min(step_tokens or self.max_step_tokens, self.max_step_tokens, max(1, total_tokens))
        out = []
        for g in self.paged:
            n = -(-total_tokens // P)
            if g.need.window is not None:
                n = min(n, -(-(g.need.window - 1 + n_step) // P) + 1)
            out.append(n)
        return out

    def close(self, rid: Hashable) -> None:
        """Give back every page and the state slot of ``rid``."""
        if rid not in self.requests:
            raise CacheError(f"request {rid!r} is not open")
        if any(r == rid for r, _ in self._in_step):
            raise CacheError(f"request {rid!r} is part of the step in flight")
        req = self.requests.pop(rid)
        n_blocks = -(-req.length // self.page_size)
        for g in self.paged:
            pages = g.held_pages(req.row, n_blocks)
            g.pool.free(pages)
            for b in range(g.first_live.pop(req.row, 0), n_blocks):
                if g.table_host[req.row, b] != NULL_PAGE:
                    g.set_entry(req.row, b, NULL_PAGE)
        self.slots.free(req.state_slot)
        self._rows.append(req.row)

    # ------------------------------------------------------------------ steps
    def begin_step(self, entries: Sequence[Tuple[Hashable, int]]) -> StepCachePlan:
        """Take pages for ``n`` new tokens of each listed request, all or nothing."""
        if self._in_step:
            raise CacheError("begin_step called while a step is in flight")
        seen = set()
        for rid, n in entries:
            if rid not in self.requests:
                raise CacheError(f"request {rid!r} is not open")
            if rid in seen:
                raise CacheError(f"request {rid!r} appears twice in one step")
            seen.add(rid)
            if n < 1:
                raise CacheError(f"request {rid!r}: a step needs at least one token")
            if self.requests[rid].length + n > self.max_seq_len:
                raise CacheError(
                    f"request {rid!r} would reach {self.requests[rid].length + n} tokens, "
                    f"the engine's longest sequence is {self.max_seq_len}")
        for g in self.paged:
            want = 0
            for rid, n in entries:
                r = self.requests[rid]
                # a windowed group frees what the *previous* length made dead before it takes more
                want += self.pages_for(r.length, n, g, g.first_live[r.row])
            reclaim = 0
            if g.need.window is not None:
                for rid, n in entries:
                    r = self.requests[rid]
                    reclaim += max(0, min(g.dead_blocks(r.length), -(-r.length // self.page_size))
                                   - g.first_live[r.row])
            if want > g.pool.free_count + reclaim:
                raise CacheError(
                    f"out of pages in cache group {g.index}: the step needs {want}, "
                    f"{g.pool.free_count + reclaim} are free of {g.pool.num_pages}")
        total = sum(n for _, n in entries)
        plan = StepCachePlan([], [], [], [], [np.empty(total, dtype=np.int32) for _ in self.paged])
        t0 = 0
        for rid, n in entries:
            r = self.requests[rid]
            plan.rows.append(r.row)
            plan.kv_lens.append(r.length + n)
            plan.state_slots.append(r.state_slot)
            plan.fresh.append(r.length == 0)
            pos = np.arange(r.length, r.length + n)
            for g in self.paged:
                self._release_dead(g, r)
                have = max(-(-r.length // self.page_size), g.first_live[r.row])
                want = -(-(r.length + n) // self.page_size)
                if want > have:
                    for b, p in zip(range(have, want), g.pool.alloc(want - have)):
                        g.set_entry(r.row, b, p)
                pages = g.table_host[r.row, pos // self.page_size].astype(np.int64)
                slots = pages * self.page_size + pos % self.page_size
                # positions whose page a window already passed (long prompt portions) are not stored
                slots[pages == NULL_PAGE] = -1
                plan.slot_maps[g.index][t0:t0 + n] = slots
            r.reserved = n
            t0 += n
        self._in_step = list(entries)
        return plan

    def _release_dead(self, g: PagedGroup, r: _Request) -> None:
        if g.need.window is None:
            return
        dead = min(g.dead_blocks(r.length), -(-r.length // self.page_size))
        first = g.first_live[r.row]
        if dead > first:
            pages = [int(p) for p in g.table_host[r.row, first:dead] if p != NULL_PAGE]
            g.pool.free(pages)
            for b in range(first, dead):
                if g.table_host[r.row, b] != NULL_PAGE:
                    g.set_entry(r.row, b, NULL_PAGE)
            g.first_live[r.row] = dead

    def end_step(self) -> None:
        """The step ran: the new tokens now count, and windows move on."""
        for rid, n in self._in_step:
            r = self.requests[rid]
            r.length += n
            r.reserved = 0
            for g in self.paged:
                self._release_dead(g, r)
        self._in_step = []

    def abort_step(self) -> None:
        """The step did not run: give back the pages taken for it."""
        for rid, n in self._in_step:
            r = self.requests[rid]
            have = -(-r.length // self.page_size)
            want = -(-(r.length + n) // self.page_size)
            for g in self.paged:
                lo = max(have, g.first_live[r.row])
                pages = [int(p) for p in g.table_host[r.row, lo:want] if p != NULL_PAGE]
                g.pool.free(pages)
                for b in range(lo, want):
                    if g.table_host[r.row, b] != NULL_PAGE:
                        g.set_entry(r.row, b, NULL_PAGE)
            r.reserved = 0
        self._in_step = []

    def take_updates(self, group: int) -> List[Tuple[int, int]]:
        """Block-table changes since the last call, as (flat index, page), oldest first."""
        g = self.paged[group]
        out, g.updates = g.updates, []
        return out

    # ------------------------------------------------------------------ invariants
    def check(self) -> None:
        """No page lost, held twice or freed twice; no slot lost; rows accounted for."""
        for g in self.paged:
            held: List[int] = []
            for rid, r in self.requests.items():
                n_blocks = -(-(r.length + r.reserved) // self.page_size)
                held += g.held_pages(r.row, n_blocks)
                if np.any(g.table_host[r.row, n_blocks:] != NULL_PAGE):
                    raise CacheError(f"request {rid!r} holds pages beyond its length")
                first = g.first_live[r.row]
                if np.any(g.table_host[r.row, :first] != NULL_PAGE):
                    raise CacheError(f"request {rid!r} holds pages its window has passed")
                if np.any(g.table_host[r.row, first:n_blocks] == NULL_PAGE):
                    raise CacheError(f"request {rid!r} misses a page inside its length")
            g.pool.check(held)
            live_rows = {r.row for r in self.requests.values()}
            for row in range(self.max_requests):
                if row not in live_rows and np.any(g.table_host[row] != NULL_PAGE):
                    raise CacheError(f"block-table row {row} holds pages but belongs to nobody")
        self.slots.check([r.state_slot for r in self.requests.values()])
        rows = [r.row for r in self.requests.values()]
        if len(set(rows)) != len(rows) or len(rows) + len(self._rows) != self.max_requests:
            raise CacheError("request rows lost or held twice")
