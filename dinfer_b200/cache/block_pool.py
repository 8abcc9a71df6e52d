"""A pool of cache pages (blocks of ``block_size`` tokens) and a table of fixed-size state slots.

Pure bookkeeping on the host; the device tensors that the ids index live with the step function.
A freed page goes on top of the free stack and is the next one handed out, so pages are used
again as early as possible (the reference frees unhashed blocks to the head of its free list and
allocates from the head: crates/core/src/kv/block_pool.rs:128-182).  There is no prefix cache
here, so a page has at most one holder.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional


class PoolError(RuntimeError):
    """A page freed twice, freed while not held, or asked for beyond what is free."""


class BlockPool:
    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise ValueError("a pool needs at least one block")
        self.num_blocks = num_blocks
        self._free: List[int] = list(range(num_blocks - 1, -1, -1))   # stack, block 0 on top
        self._held = [False] * num_blocks

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of blocks")
        if n > len(self._free):
            raise PoolError(f"asked for {n} blocks, {len(self._free)} free")
        out = []
        for _ in range(n):
            b = self._free.pop()
            self._held[b] = True
            out.append(b)
        return out

    def free(self, blocks) -> None:
        for b in blocks:
            if not (0 <= b < self.num_blocks):
                raise PoolError(f"block {b} is not of this pool")
            if not self._held[b]:
                raise PoolError(f"block {b} freed while not held")
            self._held[b] = False
            self._free.append(b)

    def is_held(self, b: int) -> bool:
        return self._held[b]


class StateSlots:
    """``max_slots`` fixed-size per-request state slots.  A request gets its slot with its first
    pages and gives it back with them; a slot handed out is reported fresh exactly once, so the
    mixer that owns the state zeroes it before first use (the reference's StateSlotTable leaves the
    zeroing to the caller too: crates/layers/src/exec.rs:251-333)."""

    def __init__(self, max_slots: int):
        self.max_slots = max_slots
        self._free = list(range(max_slots - 1, -1, -1))
        self._slot: Dict[Hashable, int] = {}
        self._fresh: Dict[Hashable, bool] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self, req: Hashable) -> Optional[int]:
        if req in self._slot:
            return self._slot[req]
        if not self._free:
            return None
        s = self._free.pop()
        self._slot[req] = s
        self._fresh[req] = True
        return s

    def slot(self, req: Hashable) -> int:
        return self._slot[req]

    def take_fresh(self, req: Hashable) -> bool:
        """True the first time it is asked after the slot was handed out."""
        f = self._fresh.get(req, False)
        self._fresh[req] = False
        return f

    def release(self, req: Hashable) -> None:
        s = self._slot.pop(req, None)
        self._fresh.pop(req, None)
        if s is not None:
            self._free.append(s)

    def holders(self):
        return dict(self._slot)
