"""Recurrent-state storage beside the paged KV cache: fixed-size per-sequence state lives in *slots*, one slot per live sequence,
handed out and taken back like KV blocks.  The reference keeps the analogous Mamba state pool next to its block engine
(src/scheduler/block_engine.rs, "mamba" snapshots); here a slot is an ``int`` and the pool a FIFO free list, the same
representation ``BlockManager`` uses for blocks.

A slot is NOT cleared when it changes hands: every kernel that reads state is told whether its entry starts a sequence
(``seq_start == 0``) and then ignores what the slot holds.
"""
from __future__ import annotations

from collections import deque
from typing import Dict, List, Sequence, Tuple

import torch

from ._lib import BackendError


class SlotPool:
    def __init__(self, num_slots: int):
        self.num_slots = int(num_slots)
        self._free: "deque[int]" = deque(range(self.num_slots))
        self._owner: Dict[int, int] = {}            # sequence id -> slot

    def num_free(self) -> int:
        return len(self._free)

    def has(self, seq_id: int) -> bool:
        return seq_id in self._owner

    def slot_of(self, seq_id: int) -> int:
        return self._owner[seq_id]

    def acquire(self, seq_id: int) -> int:
        if seq_id in self._owner:
            return self._owner[seq_id]
        if not self._free:
            raise BackendError("out of state slots")
        s = self._free.popleft()
        self._owner[seq_id] = s
        return s

    def release(self, seq_id: int) -> None:
        s = self._owner.pop(seq_id, None)
        if s is not None:
            self._free.append(s)


class StateCache:
    """Device tensors of the recurrent layers: for layer run i a tuple of tensors whose leading dimension is the slot.
    ``shapes[i]`` = tuple of per-slot shapes (e.g. ((taps - 1, channels), (heads, dk, dv))), f32 unless an entry is a (shape, dtype) pair
    (integer state such as a sequence's last token)."""

    def __init__(self, shapes: Sequence[Sequence[Tuple[int, ...]]], num_slots: int, device="cuda"):
        self.num_slots = int(num_slots)
        self.pool = SlotPool(num_slots)
        self.scratch_slot = self.num_slots          # one slot past the pool: a place for warm-up steps to write
        typed = lambda s: (tuple(s[0]), s[1]) if len(s) == 2 and isinstance(s[1], torch.dtype) else (tuple(s), torch.float32)
        self.tensors: List[Tuple[torch.Tensor, ...]] = [
            tuple(torch.zeros((self.num_slots + 1,) + typed(s)[0], dtype=typed(s)[1], device=device) for s in per_layer) for per_layer in shapes]

    def bytes_per_slot(self) -> int:
        return sum(t[0].numel() * t.element_size() for per in self.tensors for t in per)
