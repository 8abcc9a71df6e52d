"""The cache manager: block tables per request, for every group of layers.

Layers whose caches live and die together form a group: all full-attention layers one, all layers
with the same window another.  Each group has pages of its own (its own pool); within a group one
block table per request serves every layer, since each layer has its own device tensor indexed by
the same page ids.  Entry ``i`` of a table covers the positions ``[i*block_size, (i+1)*block_size)``
(a group may have a page size of its own, ``GroupSpec.block_size``); a page a window has passed is given back at
once and its entry becomes -1.

Allocation is all-or-nothing over the groups and leaves the state untouched when it fails, like
the reference's ``allocate_slots`` (crates/core/src/kv/manager.rs:203-281); ``free`` gives
pages back last-first (manager.rs:337-345).  Beside the pages every request holds one slot for
state of fixed size (used by mixers that keep such state; a Qwen3 model has none).

Prefix cache (optional; only for groups that keep every key): a full page whose keys are in the
cache is registered under a hash chained over the token ids of the request up to and including that
page.  ``begin`` gives a new request the pages of the longest chain of its tokens that every group
still has, never including the request's last token, so that at least one token is run and yields
logits (manager.rs:147-155).  Shared pages are only read: a request writes at positions behind its hit.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from .block_pool import BlockPool, PoolError, StateSlots


@dataclass(frozen=True)
class GroupSpec:
    """``window`` None: every token's keys are kept; else the last ``window`` (the token itself counts).
    ``block_size`` None: the manager's page size; else this group's own."""
    window: Optional[int] = None
    block_size: Optional[int] = None


@dataclass
class _Held:
    tables: List[List[int]]           # per group: page id per block index, -1 = released / not held
    num_tokens: int = 0               # tokens the pages cover (allocated for)
    num_computed: int = 0             # tokens whose keys are in the cache
    capacity: int = 0                 # tokens the pages of every group cover (the shortest table)
    tokens: List[int] = field(default_factory=list)      # prefix cache: the ids of the computed tokens
    hashes: List[bytes] = field(default_factory=list)    # prefix cache: chained hash per full page so far


def chain_hash(parent: bytes, tokens: Sequence[int]) -> bytes:
    """Hash of a page's contents given the hash of the page before it (16 bytes of BLAKE2b)."""
    h = hashlib.blake2b(parent, digest_size=16)
    h.update(b"".join(int(t).to_bytes(4, "little", signed=True) for t in tokens))
    return h.digest()


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], block_size: int, num_blocks: Sequence[int] | int,
                 max_num_seqs: int, enable_prefix_caching: bool = False):
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self.groups = list(groups)
        if enable_prefix_caching and any(g.window is not None for g in self.groups):
            raise ValueError("the prefix cache needs groups that keep every key (no window)")
        self.prefix_caching = bool(enable_prefix_caching)
        self.prefix_queries = 0           # tokens asked for / found by begin()
        self.prefix_hits = 0
        self.block_size = block_size                       # the default; ``block_sizes[g]`` is what group g uses
        self.block_sizes = [int(g.block_size) if g.block_size else block_size for g in self.groups]
        if any(b <= 0 for b in self.block_sizes):
            raise ValueError("a group's block_size must be positive")
        if enable_prefix_caching and len(set(self.block_sizes)) > 1:
            raise ValueError("the prefix cache needs one page size for all groups (a page's hash names its tokens)")
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
        return first_pos // self.block_sizes[group]

    def _need(self, held: Optional[_Held], total_tokens: int) -> List[int]:
        """New pages each group needs so that the request covers ``total_tokens`` tokens."""
        need = []
        for g, bs in enumerate(self.block_sizes):
            have = len(held.tables[g]) if held else 0
            need.append(max(0, (total_tokens + bs - 1) // bs - have))
        return need

    def can_allocate(self, req: Hashable, total_tokens: int) -> bool:
        held = self._reqs.get(req)
        if held is None and self.state_slots.num_free == 0:
            return False
        return all(n <= p.num_free for n, p in zip(self._need(held, total_tokens), self.pools))

    def can_allocate_all(self, wanted: Sequence) -> bool:
        """Whether every ``(request, total_tokens)`` of ``wanted`` can be allocated together (a step's batch:
        asked before any of them is, so that a step that does not fit changes nothing)."""
        need = [0] * len(self.groups)
        new = 0
        for req, total in wanted:
            held = self._reqs.get(req)
            new += held is None
            if held is not None and total <= held.capacity:
                continue
            for g, n in enumerate(self._need(held, total)):
                need[g] += n
        return new <= self.state_slots.num_free and all(n <= p.num_free for n, p in zip(need, self.pools))

    # ---- changes
    def begin(self, req: Hashable, token_ids: Sequence[int]) -> int:
        """A request enters with these tokens: take the pages of their longest cached prefix (whole
        pages, every group, never the last token) and return how many tokens they cover.  0 without
        the prefix cache, for a request that already holds pages, or when no state slot is free."""
        if not self.prefix_caching or req in self._reqs:
            return 0
        bs = self.block_sizes[0]                          # the same for all groups with the prefix cache on
        limit = (len(token_ids) - 1) // bs             # full pages that leave the last token out
        self.prefix_queries += len(token_ids)
        chain: List[bytes] = []
        found: List[List[int]] = [[] for _ in self.groups]
        parent = b""
        for i in range(limit):
            parent = chain_hash(parent, token_ids[i * bs:(i + 1) * bs])
            pages = [p.lookup(parent) for p in self.pools]
            if any(b is None for b in pages):
                break
            chain.append(parent)
            for g, b in enumerate(pages):
                found[g].append(b)
        n = len(chain)
        if n == 0:
            return 0
        if self.state_slots.acquire(req) is None:
            return 0
        for g, pool in enumerate(self.pools):
            for b in found[g]:
                pool.touch(b)
        self._reqs[req] = _Held(tables=found, num_tokens=n * bs, num_computed=n * bs, capacity=n * bs,
                                tokens=list(token_ids[:n * bs]), hashes=chain)
        self.prefix_hits += n * bs
        return n * bs

    def allocate(self, req: Hashable, total_tokens: int) -> bool:
        """Grow the request's tables to cover ``total_tokens`` tokens.  False (and nothing changed)
        when some group lacks pages or no state slot is free."""
        held = self._reqs.get(req)
        if held is not None and total_tokens <= held.capacity:      # the usual decode step: room on the last page
            if total_tokens > held.num_tokens:
                held.num_tokens = total_tokens
            return True
        if not self.can_allocate(req, total_tokens):
            return False
        if held is None:
            if self.state_slots.acquire(req) is None:
                return False
            held = _Held(tables=[[] for _ in self.groups])
            self._reqs[req] = held
        for g, n in enumerate(self._need(held, total_tokens)):
            held.tables[g].extend(self.pools[g].allocate(n))
        held.capacity = min(len(t) * bs for t, bs in zip(held.tables, self.block_sizes))
        held.num_tokens = max(held.num_tokens, total_tokens)
        return True

    def advance(self, req: Hashable, num_computed: int, new_tokens: Optional[Sequence[int]] = None) -> None:
        """The cache now holds the keys of the first ``num_computed`` tokens: give back the pages
        that every window has passed.  With the prefix cache, ``new_tokens`` are the ids of the tokens
        computed since the last call; pages they fill become findable.  An id that is not known yet (negative: a
        token the device still holds, see ``resolve``) may stand at the end of them."""
        held = self._reqs[req]
        if num_computed > held.num_tokens:
            raise PoolError(f"request {req!r}: {num_computed} tokens computed but pages cover {held.num_tokens}")
        if self.prefix_caching and new_tokens is not None:
            known = [int(t) for t in new_tokens]
            while known and known[-1] < 0:
                known.pop()
            if any(t < 0 for t in known):
                raise PoolError(f"request {req!r}: an unknown token before a known one")
            behind = len(held.tokens) + len(new_tokens) - num_computed     # tokens earlier calls left unknown
            if behind > 0 or (behind < 0 and known):
                raise PoolError(f"request {req!r}: {len(held.tokens)} known + {len(new_tokens)} new tokens "
                                f"do not make {num_computed}")
            held.tokens.extend(known)
            held.num_computed = num_computed
            self._hash_full_pages(held)
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

    def resolve(self, req: Hashable, tokens: Sequence[int]) -> None:
        """The ids of tokens that ``advance`` was told of as unknown, in order, now that the host has read them."""
        held = self._reqs.get(req)
        if held is None or not self.prefix_caching:
            return
        if len(held.tokens) + len(tokens) > held.num_computed:
            raise PoolError(f"request {req!r}: more tokens resolved than were computed")
        held.tokens.extend(int(t) for t in tokens)
        self._hash_full_pages(held)

    def _hash_full_pages(self, held: _Held) -> None:
        """Pages whose tokens are all computed and known get their hash (and become findable)."""
        bs = self.block_sizes[0]
        ready = min(len(held.tokens), held.num_computed)
        while (len(held.hashes) + 1) * bs <= ready:
            i = len(held.hashes)
            h = chain_hash(held.hashes[-1] if held.hashes else b"", held.tokens[i * bs:(i + 1) * bs])
            held.hashes.append(h)
            for g, pool in enumerate(self.pools):
                pool.set_hash(held.tables[g][i], h)     # stays unhashed if another page holds these contents

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
            seen: Dict[int, list] = {}
            for req, held in self._reqs.items():
                for i, b in enumerate(held.tables[g]):
                    if b < 0:
                        continue
                    if b in seen and not self.prefix_caching:
                        raise AssertionError(f"group {g}: page {b} held by {seen[b][0]!r} and {req!r}")
                    if b in seen and (i >= len(held.hashes) or pool.hash_of(b) != held.hashes[i]):
                        raise AssertionError(f"group {g}: page {b} shared by {seen[b]!r} and {req!r} without a common hash")
                    if not pool.is_held(b):
                        raise AssertionError(f"group {g}: page {b} of {req!r} is marked free")
                    seen.setdefault(b, []).append(req)
            for b, holders in seen.items():
                if pool.refcount(b) != len(holders):
                    raise AssertionError(f"group {g}: page {b} has {pool.refcount(b)} references, {len(holders)} holders")
            if len(seen) + pool.num_free != pool.num_blocks:
                raise AssertionError(f"group {g}: {len(seen)} held + {pool.num_free} free != {pool.num_blocks}")
            pool.check()
        holders = self.state_slots.holders()
        if set(holders) != set(self._reqs):
            raise AssertionError("state slots and page holders differ")
        if len(set(holders.values())) != len(holders):
            raise AssertionError("a state slot is held twice")
