"""Slots of fixed-size per-request state.

The reference keeps such state in a Python dict on the sequence (``kv_handle`` with the slot and
rope_delta, omniserve/runners/multimodal.py:196,215) and in a device array of lengths
(omniserve/cache/kv_prealloc.py:38-39).  Here every field is a device tensor with one row per
slot; a request holds one slot from admission to its end.  The M-RoPE cursor and rope_delta live
here; a mixer with recurrent state would keep it here too.
"""

from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch


class OutOfSlots(RuntimeError):
    pass


class StateSlots:
    def __init__(self, num_slots: int, fields: Dict[str, Tuple[Tuple[int, ...], torch.dtype]], device,
                 allocate: bool = True, spare: int = 0):
        """``spare`` further slots (numbered from ``num_slots`` on) are handed out only on request and are not
        counted as free: for rows that are no requests (what pads a decode step to the batch size of a graph)."""
        self.num_slots = int(num_slots)
        self.num_spare = int(spare)
        self.fields = dict(fields)
        self.device = device
        total = self.num_slots + self.num_spare
        self._free: List[int] = list(range(self.num_slots - 1, -1, -1))
        self._spare_free: List[int] = list(range(total - 1, self.num_slots - 1, -1))
        self._held = [False] * total
        self.tensors: Dict[str, torch.Tensor] = {}
        if allocate:
            for name, (shape, dtype) in self.fields.items():
                self.tensors[name] = torch.zeros((total,) + tuple(shape), dtype=dtype, device=device)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, spare: bool = False) -> int:
        """A free slot with every field's row zeroed."""
        pool = self._spare_free if spare else self._free
        if not pool:
            raise OutOfSlots("no free request slot")
        s = pool.pop()
        self._held[s] = True
        for t in self.tensors.values():
            t[s].zero_()
        return s

    def free(self, slot: int) -> None:
        if not (0 <= slot < self.num_slots + self.num_spare) or not self._held[slot]:
            raise ValueError(f"slot {slot} freed twice (or never handed out)")
        self._held[slot] = False
        (self._free if slot < self.num_slots else self._spare_free).append(slot)

    def write(self, name: str, slot: int, values: Sequence) -> None:
        t = self.tensors[name]
        t[slot].copy_(torch.tensor(values, dtype=t.dtype).reshape(t.shape[1:]))
