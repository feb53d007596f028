"""Slots for per-request state of fixed size.

Each live request owns one slot index from admission to finish.  The index addresses the
request's row in every persistent per-request table: the block tables of the cache groups
and the state tensors ``[num_slots, ...]`` of mixers that declare a ``StateSpec``.  The
reference has no counterpart; its only per-request runner state is the batch row
(kvcore/model/input_batch.py:65-111).
"""
from __future__ import annotations


class StateSlotError(RuntimeError):
    pass


class StateSlotPool:
    def __init__(self, num_slots: int) -> None:
        if num_slots <= 0:
            raise ValueError(f"num_slots must be positive, got {num_slots}")
        self.num_slots = int(num_slots)
        self._free = list(range(self.num_slots - 1, -1, -1))  # pop() hands out 0 first
        self._owner: list[str | None] = [None] * self.num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, owner: str) -> int:
        if not self._free:
            raise StateSlotError("no free state slot")
        slot = self._free.pop()
        self._owner[slot] = owner
        return slot

    def free(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or self._owner[slot] is None:
            raise StateSlotError(f"state slot {slot} is not held")
        self._owner[slot] = None
        self._free.append(slot)

    def owner(self, slot: int) -> str | None:
        return self._owner[slot]


__all__ = ["StateSlotError", "StateSlotPool"]
