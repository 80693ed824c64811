"""Slots for per-request state of fixed size.

One slot per live request; slot 0 is a sink that padded rows may write to and nobody
reads.  Freed slots are reused last-in first-out, and a request's first step is flagged
fresh so that mixers start from zero state instead of a previous owner's.  Same contract
as the reference's ``LinearStatePool`` (python/freetoken/kvcache/linear_state_pool.py:32-183).
"""

from __future__ import annotations

from typing import List

from ..errors import CacheError


class StateSlotPool:
    def __init__(self, num_slots: int):
        """``num_slots`` usable slots, ids 1..num_slots (0 is the sink)."""
        if num_slots < 1:
            raise CacheError(f"a state pool needs at least one slot, got {num_slots}")
        self.num_slots = num_slots
        self._free: List[int] = list(range(num_slots, 0, -1))
        self._held = [False] * (num_slots + 1)

    @property
    def free_count(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"out of state slots ({self.num_slots} in use)")
        s = self._free.pop()
        self._held[s] = True
        return s

    def free(self, slot: int) -> None:
        if not 1 <= slot <= self.num_slots or not self._held[slot]:
            raise CacheError(f"state slot {slot} freed twice or never taken")
        self._held[slot] = False
        self._free.append(slot)

    def check(self, held: List[int]) -> None:
        if len(set(held)) != len(held):
            raise CacheError("a state slot is held twice")
        if len(held) + len(self._free) != self.num_slots:
            raise CacheError("state slots lost")
