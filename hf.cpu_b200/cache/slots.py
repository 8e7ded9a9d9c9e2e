"""Slots for per-request state of fixed size.

Every live request holds one slot index.  A schedule entry whose mixer declares a
:class:`StateSpec` gets a tensor ``[max_requests, *shape]``; a request's row is zeroed when the
slot is handed out.  The reference's per-sequence state is a host struct (``gseq``,
src/ops.c:609-619) and the position counter in the context (src/model.c:200); recurrent layer
state exists there only as design notes (docs/DESIGN-SPACE.md:105, :125).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..parts.base import StateSpec


class OutOfSlots(RuntimeError):
    pass


class StateSlots:
    def __init__(self, entry_specs: Dict[int, StateSpec], max_requests: int, device: torch.device):
        self.max_requests = max_requests
        self._free: List[int] = list(range(max_requests - 1, -1, -1))
        self.slot_of: Dict[object, int] = {}
        self.tensors: Dict[int, torch.Tensor] = {
            entry: torch.zeros((max_requests, *spec.shape), dtype=spec.dtype, device=device)
            for entry, spec in entry_specs.items()}

    @property
    def free_count(self) -> int:
        return len(self._free)

    def bytes_per_request(self) -> int:
        return sum(t[0].numel() * t.element_size() for t in self.tensors.values())

    def acquire(self, req) -> int:
        if req in self.slot_of:
            raise ValueError(f"request {req!r} already holds a slot")
        if not self._free:
            raise OutOfSlots(f"all {self.max_requests} request slots are in use")
        s = self._free.pop()
        self.slot_of[req] = s
        for t in self.tensors.values():
            t[s].zero_()
        return s

    def release(self, req) -> None:
        self._free.append(self.slot_of.pop(req))

    def entry_state(self, entry: int) -> Optional[torch.Tensor]:
        return self.tensors.get(entry)

    def check(self) -> None:
        held = list(self.slot_of.values())
        assert len(held) == len(set(held)), "a slot is held twice"
        assert sorted(held + self._free) == list(range(self.max_requests)), "a slot is lost or free twice"
