"""Slots for per-request state of fixed size.

A request gets one slot index at its first step; every fixed-state layer keeps that
request's state at that index.  The reference allocates such state per session as
separate zero-filled device buffers (crates/shiso-engine/src/sessions.rs:90-116);
here it is one pool of equal slots, reused when a request ends.
"""

from __future__ import annotations

from collections import deque

from .pages import OutOfPages


class SlotPool:
    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError(f"a slot pool needs at least one slot, got {num_slots}")
        self.num_slots = num_slots
        self._free = deque(range(num_slots))
        self._held = [False] * num_slots

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages(1, 0, "state slots")
        slot = self._free.popleft()
        self._held[slot] = True
        return slot

    def give_back(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise RuntimeError(f"state slot {slot} was given back twice or never taken")
        self._held[slot] = False
        self._free.append(slot)

    def check(self) -> None:
        free = list(self._free)
        if len(set(free)) != len(free):
            raise RuntimeError("a state slot is on the free list twice")
        for s in range(self.num_slots):
            if self._held[s] == (s in self._free):
                raise RuntimeError(f"state slot {s} is both held and free, or neither")
