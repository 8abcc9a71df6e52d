"""The cache manager: block tables per request, for every group of layers.

Layers whose caches live and die together form a group: all full-attention layers one, all layers
with the same window another.  Each group has pages of its own (its own pool); within a group one
block table per request serves every layer, since each layer has its own device tensor indexed by
the same page ids.  Entry ``i`` of a table covers the positions ``[i*block_size, (i+1)*block_size)``;
a page a window has passed is given back at once and its entry becomes -1.

Allocation is all-or-nothing over the groups and leaves the state untouched when it fails, like
the reference's ``allocate_slots`` (crates/core/src/kv/manager.rs:203-281); ``free`` gives
pages back last-first (manager.rs:337-345).  Beside the pages every request holds one slot for
state of fixed size (used by mixers that keep such state; a Qwen3 model has none).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from .block_pool import BlockPool, PoolError, StateSlots


@dataclass(frozen=True)
class GroupSpec:
    """``window`` None: every token's keys are kept; else the last ``window`` (the token itself counts)."""
    window: Optional[int] = None


@dataclass
class _Held:
    tables: List[List[int]]           # per group: page id per block index, -1 = released / not held
    num_tokens: int = 0               # tokens the pages cover (allocated for)
    num_computed: int = 0             # tokens whose keys are in the cache


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], block_size: int, num_blocks: Sequence[int] | int,
                 max_num_seqs: int):
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self.groups = list(groups)
        self.block_size = block_size
        if isinstance(num_blocks, int):
            num_blocks = [num_blocks] * len(self.groups)
        if len(num_blocks) != len(self.groups):
            raise ValueError("one pool size per group")
        self.pools = [BlockPool(n) for n in num_blocks]
        self.state_slots = StateSlots(max_num_seqs)
        self._reqs: Dict[Hashable, _Held] = {}

    # ---- questions
    def __contains__(self, req: Hashable) -> bool:
        return req in self._reqs

    def requests(self):
        return list(self._reqs)

    def num_tokens(self, req: Hashable) -> int:
        return self._reqs[req].num_tokens

    def num_computed(self, req: Hashable) -> int:
        return self._reqs[req].num_computed

    def block_table(self, req: Hashable, group: int) -> List[int]:
        return self._reqs[req].tables[group]

    def num_free_blocks(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def _first_needed_block(self, group: int, num_computed: int) -> int:
        w = self.groups[group].window
        if w is None:
            return 0
        first_pos = max(0, num_computed - w + 1)      # oldest key a query at num_computed still sees
        return first_pos // self.block_size

    def _need(self, held: Optional[_Held], total_tokens: int) -> List[int]:
        """New pages each group needs so that the request covers ``total_tokens`` tokens."""
        bs = self.block_size
        want = (total_tokens + bs - 1) // bs
        need = []
        for g in range(len(self.groups)):
            have = len(held.tables[g]) if held else 0
            need.append(max(0, want - have))
        return need

    def can_allocate(self, req: Hashable, total_tokens: int) -> bool:
        held = self._reqs.get(req)
        if held is None and self.state_slots.num_free == 0:
            return False
        return all(n <= p.num_free for n, p in zip(self._need(held, total_tokens), self.pools))

    # ---- changes
    def allocate(self, req: Hashable, total_tokens: int) -> bool:
        """Grow the request's tables to cover ``total_tokens`` tokens.  False (and nothing changed)
        when some group lacks pages or no state slot is free."""
        if not self.can_allocate(req, total_tokens):
            return False
        held = self._reqs.get(req)
        if held is None:
            if self.state_slots.acquire(req) is None:
                return False
            held = _Held(tables=[[] for _ in self.groups])
            self._reqs[req] = held
        for g, n in enumerate(self._need(held, total_tokens)):
            held.tables[g].extend(self.pools[g].allocate(n))
        held.num_tokens = max(held.num_tokens, total_tokens)
        return True

    def advance(self, req: Hashable, num_computed: int) -> None:
        """The cache now holds the keys of the first ``num_computed`` tokens: give back the pages
        that every window has passed."""
        held = self._reqs[req]
        if num_computed > held.num_tokens:
            raise PoolError(f"request {req!r}: {num_computed} tokens computed but pages cover {held.num_tokens}")
        held.num_computed = num_computed
        for g in range(len(self.groups)):
            if self.groups[g].window is None:
                continue
            table = held.tables[g]
            stop = min(self._first_needed_block(g, num_computed), len(table))
            gone = [i for i in range(stop) if table[i] >= 0]
            self.pools[g].free([table[i] for i in gone])
            for i in gone:
                table[i] = -1

    def free(self, req: Hashable) -> None:
        """The request ends (or is preempted): all its pages and its state slot go back."""
        held = self._reqs.pop(req, None)
        if held is None:
            raise PoolError(f"request {req!r} holds nothing")
        for g, table in enumerate(held.tables):
            self.pools[g].free([b for b in reversed(table) if b >= 0])
        self.state_slots.release(req)

    # ---- for tests
    def check_invariants(self) -> None:
        """No page lost or held twice: per group, held pages + free pages = the pool, disjoint."""
        for g, pool in enumerate(self.pools):
            seen = {}
            for req, held in self._reqs.items():
                for b in held.tables[g]:
                    if b < 0:
                        continue
                    if b in seen:
                        raise AssertionError(f"group {g}: page {b} held by {seen[b]!r} and {req!r}")
                    if not pool.is_held(b):
                        raise AssertionError(f"group {g}: page {b} of {req!r} is marked free")
                    seen[b] = req
            if len(seen) + pool.num_free != pool.num_blocks:
                raise AssertionError(f"group {g}: {len(seen)} held + {pool.num_free} free != {pool.num_blocks}")
        holders = self.state_slots.holders()
        if set(holders) != set(self._reqs):
            raise AssertionError("state slots and page holders differ")
        if len(set(holders.values())) != len(holders):
            raise AssertionError("a state slot is held twice")
