"""A pool of cache pages (blocks of ``block_size`` tokens) and a table of fixed-size state slots.

Pure bookkeeping on the host; the device tensors that the ids index live with the step function.
Every page has a reference count; a page nobody holds is on the free list.  The free list is kept
in the order of use: a page that carries no content hash goes to its HEAD when freed and is the
next one handed out (pages are used again as early as possible); a page that carries the hash of
its contents (prefix cache) goes to the TAIL, so it stays findable as long as possible and is
evicted, least recently used first, only when the pages before it are gone.  A page taken from the
free list for new contents loses its hash.  A prefix hit takes a page out of the free list again
(crates/core/src/kv/block_pool.rs:1-8,128-182).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Hashable, List, Optional


class PoolError(RuntimeError):
    """A page freed twice, freed while not held, or asked for beyond what is free."""


class BlockPool:
    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise ValueError("a pool needs at least one block")
        self.num_blocks = num_blocks
        self._free: "OrderedDict[int, None]" = OrderedDict((b, None) for b in range(num_blocks))  # head first
        self._refs = [0] * num_blocks
        self._hash: List[Optional[bytes]] = [None] * num_blocks
        self._cached: Dict[bytes, int] = {}           # content hash -> the page that holds it
        self.evictions = 0

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
            b, _ = self._free.popitem(last=False)     # the head
            h = self._hash[b]
            if h is not None:                          # its old contents can no longer be found
                del self._cached[h]
                self._hash[b] = None
                self.evictions += 1
            self._refs[b] = 1
            out.append(b)
        return out

    def free(self, blocks) -> None:
        """One holder of each of these pages lets go; a page without holders joins the free list."""
        for b in blocks:
            if not (0 <= b < self.num_blocks):
                raise PoolError(f"block {b} is not of this pool")
            if self._refs[b] <= 0:
                raise PoolError(f"block {b} freed while not held")
            self._refs[b] -= 1
            if self._refs[b] == 0:
                self._free[b] = None                   # at the tail
                if self._hash[b] is None:
                    self._free.move_to_end(b, last=False)

    def is_held(self, b: int) -> bool:
        return self._refs[b] > 0

    def refcount(self, b: int) -> int:
        return self._refs[b]

    # ---- prefix cache
    def lookup(self, h: bytes) -> Optional[int]:
        return self._cached.get(h)

    def touch(self, b: int) -> None:
        """One more holder of a page found through its hash (it may have been free)."""
        if self._refs[b] == 0:
            del self._free[b]
        self._refs[b] += 1

    def set_hash(self, b: int, h: bytes) -> bool:
        """Make the held page findable under ``h``.  False (and nothing changed) when another page
        already holds these contents or the page has a hash."""
        if self._refs[b] <= 0:
            raise PoolError(f"block {b} hashed while not held")
        if h in self._cached or self._hash[b] is not None:
            return False
        self._hash[b] = h
        self._cached[h] = b
        return True

    def hash_of(self, b: int) -> Optional[bytes]:
        return self._hash[b]

    def check(self) -> None:
        for b in range(self.num_blocks):
            if (self._refs[b] == 0) != (b in self._free):
                raise AssertionError(f"page {b}: {self._refs[b]} holders but {'on' if b in self._free else 'off'} the free list")
            h = self._hash[b]
            if h is not None and self._cached.get(h) != b:
                raise AssertionError(f"page {b} has a hash the cache does not map to it")
        for h, b in self._cached.items():
            if self._hash[b] != h:
                raise AssertionError(f"the cache maps a hash to page {b}, which does not carry it")


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
