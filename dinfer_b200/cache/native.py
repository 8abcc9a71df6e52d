"""The cache manager with its bookkeeping in C++ (``csrc/host_core.cpp``), behind the interface of
``cache.manager.CacheManager``: the same calls, answers and errors, so either serves the step function, the
scheduler and the tests.  What it buys is the per-step cost at large batches: a decode step's packed plan is written
by one native call from the native tables (``fill_decode_plan``) instead of a Python loop over the requests.

Request ids (any hashable) are mapped to the 64-bit handles the library names requests by.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int32, c_int64, c_longlong, c_void_p
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from ..csrc import build as _build
from .block_pool import PoolError
from .manager import GroupSpec

_LIB = None


def library() -> ctypes.CDLL:
    """The host-core library, built at first use like the kernel libraries (g++, no CUDA)."""
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(_build.ensure_built(["host_core"])["host_core"])
        P, I, L = c_void_p, c_int, c_int64
        sig = {
            "dh_last_error": (ctypes.c_char_p, []),
            "dh_manager_new": (P, [I, P, P, P, I, I]), "dh_manager_delete": (None, [P]),
            "dh_contains": (I, [P, L]), "dh_num_requests": (I, [P]), "dh_requests": (I, [P, P, I]),
            "dh_num_tokens": (I, [P, L]), "dh_num_computed": (I, [P, L]), "dh_table_len": (I, [P, L, I]),
            "dh_table": (I, [P, L, I, P, I]), "dh_pool_free": (I, [P, I]), "dh_pool_blocks": (I, [P, I]),
            "dh_pool_evictions": (c_longlong, [P, I]), "dh_pool_refcount": (I, [P, I, I]), "dh_pool_check": (I, [P, I]),
            "dh_prefix_queries": (c_longlong, [P]), "dh_prefix_hits": (c_longlong, [P]),
            "dh_slots_free": (I, [P]), "dh_slot": (I, [P, L]), "dh_take_fresh": (I, [P, L]),
            "dh_can_allocate": (I, [P, L, I]), "dh_can_allocate_all": (I, [P, P, P, I]), "dh_allocate": (I, [P, L, I]),
            "dh_begin": (I, [P, L, P, I]), "dh_advance": (I, [P, L, I, P, I]), "dh_resolve": (I, [P, L, P, I]),
            "dh_free": (I, [P, L]), "dh_check_invariants": (I, [P]),
            "dh_decode_plan_fill": (I, [P, P, I, I, P, P, P, I, I]), "dh_advance_many": (I, [P, P, P, I]),
        }
        for name, (res, args) in sig.items():
            f = getattr(lib, name)
            f.restype, f.argtypes = res, args
        _LIB = lib
    return _LIB


def _error(lib) -> str:
    msg = lib.dh_last_error()
    return msg.decode("utf-8", "replace") if msg else "host core error"


class _PoolView:
    """What callers read of one group's pool."""

    def __init__(self, owner: "NativeCacheManager", group: int):
        self._o, self._g = owner, group

    @property
    def num_free(self) -> int:
        return self._o._lib.dh_pool_free(self._o._h, self._g)

    @property
    def num_blocks(self) -> int:
        return self._o._lib.dh_pool_blocks(self._o._h, self._g)

    @property
    def evictions(self) -> int:
        return int(self._o._lib.dh_pool_evictions(self._o._h, self._g))

    def refcount(self, b: int) -> int:
        return self._o._lib.dh_pool_refcount(self._o._h, self._g, int(b))

    def check(self) -> None:
        if self._o._lib.dh_pool_check(self._o._h, self._g):
            raise AssertionError(_error(self._o._lib))


class _SlotsView:
    def __init__(self, owner: "NativeCacheManager"):
        self._o = owner

    @property
    def num_free(self) -> int:
        return self._o._lib.dh_slots_free(self._o._h)

    def slot(self, req: Hashable) -> int:
        s = self._o._lib.dh_slot(self._o._h, self._o._ids[req])
        if s < 0:
            raise KeyError(req)
        return s

    def take_fresh(self, req: Hashable) -> bool:
        rid = self._o._ids.get(req)
        return bool(rid is not None and self._o._lib.dh_take_fresh(self._o._h, rid))

    def holders(self) -> Dict[Hashable, int]:
        return {r: self.slot(r) for r in self._o.requests()}


class NativeCacheManager:
    def __init__(self, groups: Sequence[GroupSpec], block_size: int, num_blocks, max_num_seqs: int,
                 enable_prefix_caching: bool = False):
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self.groups = list(groups)
        if enable_prefix_caching and any(g.window is not None for g in self.groups):
            raise ValueError("the prefix cache needs groups that keep every key (no window)")
        self.prefix_caching = bool(enable_prefix_caching)
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
        if any(n <= 0 for n in num_blocks):
            raise ValueError("a pool needs at least one block")
        self._lib = library()
        windows = (c_int * len(self.groups))(*[int(g.window or 0) for g in self.groups])
        blocks = (c_int * len(self.groups))(*[int(n) for n in num_blocks])
        sizes = (c_int * len(self.groups))(*self.block_sizes)
        self._h = self._lib.dh_manager_new(len(self.groups), windows, sizes, blocks, max_num_seqs,
                                           int(self.prefix_caching))
        if not self._h:
            raise ValueError(_error(self._lib))
        self._ids: Dict[Hashable, int] = {}          # request id -> handle, for the requests that hold something
        self._names: Dict[int, Hashable] = {}
        self._next = 1
        self.pools = [_PoolView(self, g) for g in range(len(self.groups))]
        self.state_slots = _SlotsView(self)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.dh_manager_delete(h)

    # ---- handles
    def handle(self, req: Hashable) -> int:
        rid = self._ids.get(req)
        if rid is None:
            rid = self._next
            self._next += 1
            self._ids[req] = rid
            self._names[rid] = req
        return rid

    def _forget_if_gone(self, req: Hashable) -> None:
        rid = self._ids.get(req)
        if rid is not None and not self._lib.dh_contains(self._h, rid):
            del self._ids[req]
            del self._names[rid]

    # ---- questions
    def __contains__(self, req: Hashable) -> bool:
        rid = self._ids.get(req)
        return rid is not None and bool(self._lib.dh_contains(self._h, rid))

    def requests(self):
        n = self._lib.dh_num_requests(self._h)
        buf = (c_int64 * max(1, n))()
        self._lib.dh_requests(self._h, buf, n)
        return [self._names[buf[i]] for i in range(n)]

    def _held(self, req: Hashable) -> int:
        rid = self._ids.get(req)
        if rid is None or not self._lib.dh_contains(self._h, rid):
            raise KeyError(req)
        return rid

    def num_tokens(self, req: Hashable) -> int:
        return self._lib.dh_num_tokens(self._h, self._held(req))

    def num_computed(self, req: Hashable) -> int:
        return self._lib.dh_num_computed(self._h, self._held(req))

    def block_table(self, req: Hashable, group: int) -> List[int]:
        rid = self._held(req)
        n = self._lib.dh_table_len(self._h, rid, group)
        buf = (c_int32 * max(1, n))()
        self._lib.dh_table(self._h, rid, group, buf, n)
        return list(buf[:n])

    def num_free_blocks(self, group: int = 0) -> int:
        return self._lib.dh_pool_free(self._h, group)

    @property
    def prefix_queries(self) -> int:
        return int(self._lib.dh_prefix_queries(self._h))

    @property
    def prefix_hits(self) -> int:
        return int(self._lib.dh_prefix_hits(self._h))

    def can_allocate(self, req: Hashable, total_tokens: int) -> bool:
        rid = self._ids.get(req, 0)
        return bool(self._lib.dh_can_allocate(self._h, rid, int(total_tokens)))

    def can_allocate_all(self, wanted: Sequence) -> bool:
        n = len(wanted)
        rs = (c_int64 * max(1, n))(*[self._ids.get(r, -(i + 1)) for i, (r, _) in enumerate(wanted)])
        ts = (c_int * max(1, n))(*[int(t) for _, t in wanted])
        return bool(self._lib.dh_can_allocate_all(self._h, rs, ts, n))

    # ---- changes
    def begin(self, req: Hashable, token_ids: Sequence[int]) -> int:
        if not self.prefix_caching or req in self:
            return 0
        arr = np.ascontiguousarray(token_ids, dtype=np.int32)
        rid = self.handle(req)
        n = self._lib.dh_begin(self._h, rid, arr.ctypes.data, arr.size)
        if n == 0:
            self._forget_if_gone(req)
        return n

    def allocate(self, req: Hashable, total_tokens: int) -> bool:
        ok = bool(self._lib.dh_allocate(self._h, self.handle(req), int(total_tokens)))
        if not ok:
            self._forget_if_gone(req)
        return ok

    def advance(self, req: Hashable, num_computed: int, new_tokens: Optional[Sequence[int]] = None) -> None:
        rid = self._held(req)
        if new_tokens is not None and self.prefix_caching and len(new_tokens):
            arr = np.ascontiguousarray(new_tokens, dtype=np.int32)
            rc = self._lib.dh_advance(self._h, rid, int(num_computed), arr.ctypes.data, arr.size)
        else:
            rc = self._lib.dh_advance(self._h, rid, int(num_computed), None, 0)
        if rc:
            raise PoolError(_error(self._lib))

    def advance_many(self, handles: np.ndarray, computed: np.ndarray) -> None:
        """``advance`` for a step's requests at once (int64 handles, int32 token counts; without the prefix cache)."""
        if self._lib.dh_advance_many(self._h, handles.ctypes.data, computed.ctypes.data, len(handles)):
            raise PoolError(_error(self._lib))

    def resolve(self, req: Hashable, tokens: Sequence[int]) -> None:
        rid = self._ids.get(req)
        if rid is None or not self.prefix_caching:
            return
        arr = np.ascontiguousarray(tokens, dtype=np.int32)
        if self._lib.dh_resolve(self._h, rid, arr.ctypes.data, arr.size):
            raise PoolError(_error(self._lib))

    def free(self, req: Hashable) -> None:
        rid = self._ids.get(req)
        if rid is None or self._lib.dh_free(self._h, rid):
            raise PoolError(f"request {req!r} holds nothing" if rid is None else _error(self._lib))
        del self._ids[req]
        del self._names[rid]

    # ---- the packed plan of a decode-only step, written by the library from its own tables
    def fill_decode_plan(self, words: np.ndarray, bucket: int, width: int, reqs: Sequence[Hashable],
                         tokens: Sequence[int], starts: Sequence[int], spare_state_slot: int = 0) -> int:
        """``words``: the plan's int32 words (a view of pinned memory), in the layout of
        ``PlanBuilder.layout(bucket, bucket, bucket, width)``.  Returns the words written."""
        n = len(reqs)
        rs = np.fromiter((self._ids[r] for r in reqs), dtype=np.int64, count=n)
        tk = np.asarray(tokens, dtype=np.int32)
        st = np.asarray(starts, dtype=np.int32)
        used = self._lib.dh_decode_plan_fill(self._h, words.ctypes.data, bucket, width, rs.ctypes.data, tk.ctypes.data,
                                             st.ctypes.data, n, int(spare_state_slot))
        if used < 0:
            raise PoolError(_error(self._lib))
        return used

    # ---- for tests
    def check_invariants(self) -> None:
        if self._lib.dh_check_invariants(self._h):
            raise AssertionError(_error(self._lib))
