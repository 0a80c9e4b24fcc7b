"""Per-sequence state of recurrent layers, next to the paged KV cache.

A recurrent layer (linear recurrence, short convolution) carries a fixed-size state per sequence instead of a growing
list of keys.  The pool holds, for every entry a model declares (one per recurrent layer execution and kind of state),
one tensor ``[n_slots, *shape]``; a sequence owns the same slot index in all of them from its first forward until it is
flushed.  Slots are handed out by the block allocator of the KV cache (``blocked_allocator.py``) and are not cleared on
reuse: kernels treat the state of a sequence that has seen no token as zero.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Tuple

import torch

from .blocked_allocator import BlockedAllocator


@dataclass
class StatePoolConfig:
    entries: List[Tuple[Tuple[int, ...], torch.dtype]] = field(default_factory=list)     # (shape per slot, dtype)

    def add(self, shape, dtype: torch.dtype) -> int:
        self.entries.append((tuple(int(x) for x in shape), dtype))
        return len(self.entries) - 1

    def bytes_per_slot(self) -> int:
        total = 0
        for shape, dtype in self.entries:
            n = 1
            for x in shape:
                n *= x
            total += n * torch.tensor([], dtype=dtype).element_size()
        return total


class RecurrentStatePool:
    def __init__(self, config: StatePoolConfig, n_slots: int, device=None) -> None:
        dev = device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")
        self._n_slots = n_slots
        self._tensors = [torch.zeros((n_slots, *shape), dtype=dtype, device=dev) for shape, dtype in config.entries]
        self._allocator = BlockedAllocator(n_slots)

    def acquire(self) -> int:
        return int(self._allocator.allocate(1)[0])

    def release(self, slot: int) -> None:
        self._allocator.free(int(slot))

    def get(self, entry: int) -> torch.Tensor:
        return self._tensors[entry]

    @property
    def free_slots(self) -> int:
        return self._allocator.free_blocks

    @property
    def n_slots(self) -> int:
        return self._n_slots
