"""A step's batch, from the host's description to the tensors the parts read.

The host side is a list of ``StepEntry`` (request, its next tokens, the places whose logits are
wanted).  ``PlanBuilder`` flattens them request-major into one packed int32 buffer in pinned
memory, copied to the device in one transfer, and hands out views: ids, positions, cu_seqlens,
seq_lens, and per cache group the block table and the slot of every new token.  The fields follow
the reference's ``BatchPlan`` (crates/core/src/runner.rs:46-89, built at runner.rs:745-876).

For CUDA graphs a batch can be padded to a fixed number of requests with dummy rows (token 0,
position 0, no slot, length 1, no pages) and a fixed table width, so that every view keeps its
address and shape (crates/layers/src/exec.rs:226-247,392-404 does the same padding).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..parts.base import CacheGroupView, StepContext


@dataclass
class StepEntry:
    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # indices into ``tokens`` whose logits are returned


# DINFER_VALIDATE_PLANS=1: every plan is checked on the host before it goes to the device (see PlanBuilder._validate)
VALIDATE_PLANS = os.environ.get("DINFER_VALIDATE_PLANS", "0") == "1"


class OutOfPages(RuntimeError):
    """The cache pool cannot hold the tokens of this step."""


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class PlanBuilder:
    """Owns the pinned staging buffers (a small ring, so that a buffer is not rewritten while its
    copy may still be in flight) and the device buffers the views point into."""

    RING = 4

    def __init__(self, manager: CacheManager, device, max_tokens: int, max_reqs: int, max_blocks: int,
                 max_positions: Optional[int] = None, spare_state_slot: int = 0):
        self.manager = manager
        self.device = device
        self.max_blocks = max_blocks
        self.max_positions = max_positions          # rows of the position table (None: not known here)
        self.spare_state_slot = spare_state_slot    # the state slot of rows without a request (no request holds it)
        self.max_tokens, self.max_reqs = max_tokens, max_reqs
        self.capacity = self.words(max_tokens, max_reqs, max_tokens, max_blocks)
        on_gpu = torch.device(device).type == "cuda"
        self._host = [torch.empty(self.capacity, dtype=torch.int32, pin_memory=on_gpu) for _ in range(self.RING)]
        self._events = [None] * self.RING
        self._dev = [torch.empty(self.capacity, dtype=torch.int32, device=device) for _ in range(self.RING)]
        self._turn = 0
        self.h2d_bytes = 0

    def words(self, T: int, B: int, R: int, width: int) -> int:
        """int32 words of a packed plan of T tokens, B requests, R logits rows, tables ``width`` wide."""
        ng = len(self.manager.groups)
        return (2 * _align(T) + _align(R) + _align(B + 1) + 3 * _align(B)
                + ng * (_align(T) + _align(B * width)) + 16)

    def layout(self, T: int, B: int, R: int, width: int) -> Tuple[Dict[str, Tuple[int, int]], int]:
        """(offset, words) of every field of a packed plan, and the plan's length in words."""
        views: Dict[str, Tuple[int, int]] = {}
        off = 0
        fields = [("ids", T), ("pos", T), ("rows", R), ("cu", B + 1), ("seq", B), ("sslots", B), ("fresh", B)]
        for g in range(len(self.manager.groups)):
            fields += [(f"slot{g}", T), (f"tab{g}", B * width)]
        for name, n in fields:
            views[name] = (off, n)
            off = _align(off + n)
        return views, off

    def _validate(self, T, B, cu, seq, pos, rows, tables, slot_maps) -> None:
        """What every kernel takes for granted about a plan (checked on the host when DINFER_VALIDATE_PLANS=1, as
        the tests do: the device tools that would catch an access out of range are not at hand everywhere).
        Dummy requests are held to the same rules: a kernel walks their tables and looks their positions up too."""
        m = self.manager
        for g, tab in enumerate(tables):
            if B and int(seq.max()) > tab.shape[1] * m.block_sizes[g]:
                raise AssertionError(f"plan: a request of {int(seq.max())} tokens is longer than its table of "
                                     f"{tab.shape[1]} pages of group {g} covers")
        if T and self.max_positions is not None and int(pos.max()) >= self.max_positions:
            raise AssertionError(f"plan: position {int(pos.max())} is outside the position table of {self.max_positions}")
        if int(cu[0]) != 0 or int(cu[-1]) != T or np.any(np.diff(cu) < 0):
            raise AssertionError("plan: request offsets must rise from 0 to the number of tokens")
        if rows.size and (rows.min() < 0 or rows.max() >= max(T, 1)):
            raise AssertionError("plan: a logits row outside the step's tokens")
        if T and (pos.min() < 0 or np.any(pos >= np.repeat(seq, np.diff(cu)))):
            raise AssertionError("plan: a token's position is not inside its request")
        for g, (tab, sl) in enumerate(zip(tables, slot_maps)):
            n = m.pools[g].num_blocks
            if tab.min() < -1 or tab.max() >= n:
                raise AssertionError(f"plan: group {g}: a page id outside the pool of {n}")
            if T and (sl.min() < -1 or sl.max() >= n * m.block_sizes[g]):
                raise AssertionError(f"plan: group {g}: a slot outside the pool")
            live = sl[sl >= 0]
            if live.size != np.unique(live).size:
                raise AssertionError(f"plan: group {g}: two tokens of a step write the same slot")

    def _next_turn(self) -> int:
        """The next pinned buffer of the ring, once its last copy has left it."""
        k = self._turn
        self._turn = (k + 1) % self.RING
        if self._events[k] is not None:
            self._events[k].synchronize()
        return k

    def _send(self, k: int, words: int, dev: torch.Tensor) -> None:
        if words > dev.numel():
            raise ValueError("the plan does not fit its device buffer")
        dev[:words].copy_(self._host[k][:words], non_blocking=True)
        if dev.is_cuda:
            ev = self._events[k] or torch.cuda.Event()
            ev.record()
            self._events[k] = ev
        self.h2d_bytes = words * 4

    def build(self, entries: Sequence[StepEntry], starts: Sequence[int], *, pad_reqs: Optional[int] = None,
              table_width: Optional[int] = None, dev: Optional[torch.Tensor] = None,
              slots: Optional[Sequence[Tuple[int, int]]] = None):
        """``starts[i]`` = tokens of entry i already in the cache; pages must be allocated already.
        ``pad_reqs``: pad with one-token dummy requests up to this many and ask for every row's
        logits (the layout of a captured decode graph).  ``slots``: the layout of a captured graph in
        general: one ``(entry index or -1, tokens)`` per request place, in the order of the batch; a place
        without an entry is a dummy request of that many tokens (none, or tokens 0 at positions 0.. with no
        slot and no pages), and the logits of every place's last token are asked for (of token 0 for a place
        without tokens).  ``dev``: the int32 device buffer to fill (default: the next one of the ring).
        Returns (ids, logits_rows, ctx)."""
        m = self.manager
        if slots is None:
            n_pad = (pad_reqs - len(entries)) if pad_reqs is not None else 0
            if n_pad < 0:
                raise ValueError("pad_reqs below the number of requests")
            slots = [(i, len(e.tokens)) for i, e in enumerate(entries)] + [(-1, 1)] * n_pad
            every_place = pad_reqs is not None
        else:
            every_place = True
            used = sorted(i for i, _ in slots if i >= 0)
            if used != list(range(len(entries))) or any(n != len(entries[i].tokens) for i, n in slots if i >= 0):
                raise ValueError("slots must place every entry once, with its number of tokens")
        B = len(slots)
        lens = [n for _, n in slots]
        T = sum(lens)
        if T > self.max_tokens or B > self.max_reqs:
            raise ValueError(f"step of {T} tokens / {B} requests exceeds the plan buffers "
                             f"({self.max_tokens} / {self.max_reqs})")
        cu = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(lens, out=cu[1:])
        seq = np.asarray([max(1, n) for n in lens], dtype=np.int32)      # a dummy request is as long as its tokens
        ids = np.zeros(T, dtype=np.int32)
        pos = np.zeros(T, dtype=np.int32)
        rows: List[int] = []
        for j, (i, n) in enumerate(slots):
            a, b = cu[j], cu[j + 1]
            if i < 0:
                pos[a:b] = np.arange(n, dtype=np.int32)
                continue
            e = entries[i]
            seq[j] = starts[i] + n
            ids[a:b] = np.asarray(e.tokens, dtype=np.int64)
            pos[a:b] = np.arange(starts[i], starts[i] + n, dtype=np.int32)
            for w in e.want:
                if not (0 <= w < n):
                    raise ValueError(f"request {e.req_id!r}: wanted place {w} is outside its {n} tokens")
                rows.append(int(a) + int(w))
        if every_place:
            rows_np = np.asarray([max(0, int(cu[j + 1]) - 1) if lens[j] else 0 for j in range(B)], dtype=np.int32)
        else:
            rows_np = np.asarray(rows, dtype=np.int32)
        if table_width is not None:
            width = table_width
        else:
            small = min(m.block_sizes)                       # one width for all groups: what the smallest pages need
            width = max(1, max((int(s_) + small - 1) // small for s_ in seq)) if B else 1
        if width > self.max_blocks:
            raise ValueError(f"a request needs {width} pages, the plan buffers hold {self.max_blocks}")
        tables, slot_maps = [], []
        for g in range(len(m.groups)):
            bs = m.block_sizes[g]
            tab = np.full((B, width), -1, dtype=np.int32)
            sl = np.full(T, -1, dtype=np.int32)
            for j, (i, n) in enumerate(slots):
                if i < 0:
                    continue
                t = m.block_table(entries[i].req_id, g)
                k = min(len(t), width)
                tab[j, :k] = t[:k]
                p = pos[cu[j]:cu[j + 1]]
                blk = tab[j, p // bs]
                sl[cu[j]:cu[j + 1]] = np.where(blk >= 0, blk * bs + p % bs, -1)
            tables.append(tab)
            slot_maps.append(sl)
        sslots = np.full(B, self.spare_state_slot, dtype=np.int32)
        fresh = np.zeros(B, dtype=np.int32)
        for j, (i, n) in enumerate(slots):
            if i >= 0:
                sslots[j] = m.state_slots.slot(entries[i].req_id)
                fresh[j] = 1 if m.state_slots.take_fresh(entries[i].req_id) else 0
        slots_ = slot_maps

        if VALIDATE_PLANS:
            self._validate(T, B, cu, seq, pos, rows_np, tables, slot_maps)

        # pack: the order and the alignment fix every view's offset for given (T, B, R, width)
        k = self._next_turn()
        host = self._host[k].numpy()
        views, off = self.layout(T, B, rows_np.size, width)

        def put(name, arr):
            o, n = views[name]
            host[o:o + n] = arr.reshape(-1)

        put("ids", ids); put("pos", pos); put("rows", rows_np); put("cu", cu); put("seq", seq)
        put("sslots", sslots); put("fresh", fresh)
        for g in range(len(m.groups)):
            put(f"slot{g}", slots_[g]); put(f"tab{g}", tables[g])
        if dev is None:
            dev = self._dev[k]
        self._send(k, off, dev)

        def view(name):
            o, n = views[name]
            return dev[o:o + n]

        groups = [CacheGroupView(m.block_sizes[g], view(f"tab{g}").view(B, width), view(f"slot{g}"), m.groups[g].window)
                  for g in range(len(m.groups))]
        ctx = StepContext(
            num_tokens=T, num_reqs=B, positions=view("pos"), cu_seqlens=view("cu"), seq_lens=view("seq"),
            groups=groups, state_slots=view("sslots"), state_fresh=view("fresh"),
            max_q_len=max(lens) if lens else 0, max_seq_len=int(seq.max()) if B else 0,
            max_prefill_seq_len=max([int(seq[i]) for i, n in enumerate(lens) if n > 1] or [0]),
            all_decode=all(n == 1 for n in lens),
            any_decode=any(n == 1 for n in lens), any_prefill=any(n > 1 for n in lens),
            cu_seqlens_host=cu.tolist(), seq_lens_host=seq.tolist(),
            state_slots_host=sslots.tolist(), state_fresh_host=fresh.tolist())
        return view("ids"), view("rows"), ctx


class DecodePlan:
    """The packed plan of a captured decode graph, kept on the host between steps.

    A decode-only step changes little of its plan: one token, position and slot per request and,
    now and then, one more page at the end of a table.  So the host keeps the last plan of the
    graph's bucket and rewrites only that; rows whose request changed (or whose table is another
    list, as after a preemption) are written whole.  The layout is the one ``PlanBuilder.build``
    makes for ``pad_reqs=bucket`` and this table width, which the graph was captured with."""

    def __init__(self, builder: PlanBuilder, bucket: int, width: int, dev: torch.Tensor):
        self.builder, self.bucket, self.width, self.dev = builder, bucket, width, dev
        self.views, self.words = builder.layout(bucket, bucket, bucket, width)
        self.ng = len(builder.manager.groups)
        self.shadow = np.zeros(self.words, dtype=np.int32)
        f = self._field
        f("rows")[:] = np.arange(bucket, dtype=np.int32)
        f("cu")[:] = np.arange(bucket + 1, dtype=np.int32)
        f("seq")[:] = 1
        f("sslots")[:] = builder.spare_state_slot
        for g in range(self.ng):
            f(f"slot{g}")[:] = -1
            f(f"tab{g}")[:] = -1
        self._ids, self._pos, self._seq = f("ids"), f("pos"), f("seq")
        self._sslots, self._fresh = f("sslots"), f("fresh")
        self._slot = [f(f"slot{g}") for g in range(self.ng)]
        self._tab = [f(f"tab{g}").reshape(bucket, width) for g in range(self.ng)]
        self._windowed = [builder.manager.groups[g].window is not None for g in range(self.ng)]
        # per row and group: the table list last copied from, and how many of its entries
        self._src = [[None] * self.ng for _ in range(bucket)]
        self._copied = [[0] * self.ng for _ in range(bucket)]
        self._live = 0

    def _field(self, name: str) -> np.ndarray:
        o, n = self.views[name]
        return self.shadow[o:o + n]

    def _check(self) -> None:
        """The plan in ``shadow`` names pages and slots of the pools only, and no slot twice."""
        m = self.builder.manager
        for g in range(self.ng):
            n = m.pools[g].num_blocks
            live = self._slot[g][self._slot[g] >= 0]
            if self._tab[g].min() < -1 or self._tab[g].max() >= n or (live.size and live.max() >= n * m.block_sizes[g]) \
                    or live.size != np.unique(live).size:
                raise AssertionError(f"decode plan: group {g}: a page or slot outside the pool, or a slot written twice")

    def fill(self, entries: Sequence[StepEntry], starts: Sequence[int]) -> None:
        """Write the step of ``entries`` (one token each) into the plan and send it to the device."""
        b = self.builder
        m = b.manager
        n_real = len(entries)
        if n_real > self.bucket:
            raise ValueError("more requests than the graph's bucket")
        width = self.width
        if hasattr(m, "fill_decode_plan"):
            # the cache manager whose tables live in C++ writes the plan itself, straight into the pinned buffer
            k = b._next_turn()
            words = b._host[k].numpy()[:self.words]
            m.fill_decode_plan(words, self.bucket, width, [e.req_id for e in entries], [e.tokens[0] for e in entries], starts,
                               b.spare_state_slot)
            if VALIDATE_PLANS:
                self.shadow[:] = words
                self._check()
            b._send(k, self.words, self.dev)
            return
        for i, e in enumerate(entries):
            p = starts[i]
            self._ids[i] = e.tokens[0]
            self._pos[i] = p
            self._seq[i] = p + 1
            self._sslots[i] = m.state_slots.slot(e.req_id)
            self._fresh[i] = 1 if m.state_slots.take_fresh(e.req_id) else 0
            for g in range(self.ng):
                t = m.block_table(e.req_id, g)
                n = min(len(t), width)
                row = self._tab[g][i]
                if self._src[i][g] is not t or self._windowed[g]:
                    row[:n] = t[:n]
                    row[n:] = -1
                    self._src[i][g] = t
                else:
                    c = self._copied[i][g]
                    if n > c:
                        row[c:n] = t[c:n]
                self._copied[i][g] = n
                bs = m.block_sizes[g]
                blk = t[p // bs] if p // bs < n else -1
                self._slot[g][i] = blk * bs + p % bs if blk >= 0 else -1
        for i in range(n_real, self._live):           # rows that fell out of use become dummy rows
            self._ids[i] = 0
            self._pos[i] = 0
            self._seq[i] = 1
            self._sslots[i] = b.spare_state_slot
            self._fresh[i] = 0
            for g in range(self.ng):
                self._tab[g][i] = -1
                self._slot[g][i] = -1
                self._src[i][g] = None
                self._copied[i][g] = 0
        self._live = n_real
        if VALIDATE_PLANS:
            self._check()
        k = b._next_turn()
        b._host[k].numpy()[:self.words] = self.shadow
        b._send(k, self.words, self.dev)
