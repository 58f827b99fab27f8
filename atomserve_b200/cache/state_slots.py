"""Slots for per-request state of fixed size.

Every running request holds one slot id in [0, num_slots) from admission until it finishes or
is preempted. Parts that keep constant-size state per request (a recurrent mixer's state, a
sampler's counters) register a buffer `[num_slots, *shape]` here and index it by slot; a
slot's rows are zeroed when the slot is handed out, so no request sees its predecessor's
state. Qwen3's attention keeps nothing here; the slot is taken all the same, so that adding
such a part changes no engine code. (The reference keeps per-request state only on the host:
atomserve/sequence.py:60-83, atomserve/sampler.py:53-70.)
"""

from __future__ import annotations

import torch


class StateSlots:
    def __init__(self, num_slots: int, device: torch.device | str = "cpu"):
        self.num_slots = num_slots
        self.device = torch.device(device)
        self._free = list(range(num_slots - 1, -1, -1))  # pop() hands out 0 first
        self._in_use: set[int] = set()
        self.buffers: dict[str, torch.Tensor] = {}

    def register(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        if name in self.buffers:
            raise KeyError(f"state buffer {name!r} is already registered")
        self.buffers[name] = torch.zeros((self.num_slots, *shape), dtype=dtype, device=self.device)
        return self.buffers[name]

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise RuntimeError("no free state slot")
        slot = self._free.pop()
        self._in_use.add(slot)
        for buf in self.buffers.values():
            buf[slot].zero_()
        return slot

    def give_back(self, slot: int) -> None:
        if slot not in self._in_use:
            raise ValueError(f"state slot {slot} is not in use")
        self._in_use.remove(slot)
        self._free.append(slot)
