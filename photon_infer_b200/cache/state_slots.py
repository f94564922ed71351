"""Slots for per-request state of fixed size (a recurrent mixer's state, for
instance).  Every live request owns one slot index; each run-list entry whose mixer
declares a ``StateSpec`` has a tensor ``[max_sequences, *shape]`` indexed by it.  A
slot is cleared when it is handed out.  The Llama decoder has no such state; the
pool is there so that a mixer which has can be added without touching the engine.
The reference has nothing comparable.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..errors import ErrorCode, PhotonError
from ..parts.base import StateSpec


class StateSlotPool:
    def __init__(self, max_sequences: int, specs: Dict[int, StateSpec], device: Optional[torch.device]):
        self.max_sequences = max_sequences
        self._free: List[int] = list(range(max_sequences - 1, -1, -1))
        self._owner: Dict[object, int] = {}
        self.specs = dict(specs)                # run-list entry -> spec
        self.tensors: Dict[int, torch.Tensor] = {}
        if device is not None:
            for entry, s in self.specs.items():
                self.tensors[entry] = torch.zeros((max_sequences, *s.shape), dtype=s.dtype, device=device)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, rid) -> int:
        if rid in self._owner:
            raise PhotonError(ErrorCode.INVALID_STATE, f"request {rid!r} already has a state slot")
        if not self._free:
            raise PhotonError(ErrorCode.OUT_OF_MEMORY, f"all {self.max_sequences} request slots are in use")
        slot = self._free.pop()
        self._owner[rid] = slot
        for t in self.tensors.values():
            t[slot].zero_()
        return slot

    def slot_of(self, rid) -> int:
        return self._owner[rid]

    def free(self, rid) -> None:
        if rid not in self._owner:
            raise PhotonError(ErrorCode.DOUBLE_FREE, f"request {rid!r} holds no state slot")
        self._free.append(self._owner.pop(rid))

    def bytes_per_slot(self) -> int:
        total = 0
        for s in self.specs.values():
            n = 1
            for d in s.shape:
                n *= d
            total += n * torch.empty((), dtype=s.dtype).element_size()
        return total
