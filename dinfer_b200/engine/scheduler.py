"""Continuous batching above the step function.

Every step: running requests first, then waiting ones while the token budget, ``max_num_seqs`` and
the pages last.  A prompt longer than the budget is cut into portions; a request whose known tokens
are all in the cache decodes one token a step.  When pages run out the LAST running request is
preempted: its pages go back, it returns to the FRONT of the waiting queue and is recomputed from
token 0 later; a request never preempts itself while others run (it sits the step out), and a
request that alone does not fit is finished with ``length``.  Nothing is admitted in a step that
preempted.  This is the policy of the reference's scheduler (crates/core/src/sched/mod.rs:318-644
for schedule, :646-680 for the bookkeeping after it and preemption, :687-828 for the update and
the stop check), without its speculative tokens.  With the prefix cache on, a request that enters
takes over the cached pages of its beginning first.

Scheduling ahead (the reference's asynchronous scheduling, :645-668 and :700-760): ``schedule(lookahead=True)``
is called while the previous step still runs.  A request that samples in a step is then counted as one
token longer at once (``num_placeholders``: sampled on the device, not yet read), so the next step can
decode that token before the host knows it; ``update`` fills the value in when it arrives.  A request
whose token in flight is certainly its last (``max_tokens``, ``max_model_len``) is not scheduled again;
one that stops on an end-of-sequence token has run one step in vain, whose result is dropped; one that
was preempted with a token in flight still gets that token appended.

Pure host code: it owns the queues and asks the cache manager for pages; it never touches the GPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from .request import FinishReason, Request, RequestStatus


@dataclass
class ScheduledRequest:
    request: Request
    start: int            # tokens already in the cache
    num_tokens: int       # tokens run in this step
    samples: bool         # the step's last row yields the request's next token
    num_generated: int = 0    # output tokens the request had before this step, those in flight included


@dataclass
class SchedulerOutput:
    scheduled: List[ScheduledRequest] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    finished: List[Request] = field(default_factory=list)     # finished by the scheduler itself (no fit)

    @property
    def num_tokens(self) -> int:
        return sum(s.num_tokens for s in self.scheduled)


class Scheduler:
    def __init__(self, config: EngineConfig, manager: CacheManager, eos_token_ids: Sequence[int] = ()):
        self.config = config
        self.manager = manager
        self.eos = set(int(x) for x in eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.num_preemptions = 0

    # ---- queue
    def add_request(self, req: Request) -> None:
        req.params.validate()
        if not req.prompt_ids:
            raise ValueError(f"request {req.req_id!r}: empty prompt")
        if len(req.prompt_ids) >= self.config.max_model_len:
            raise ValueError(f"request {req.req_id!r}: prompt of {len(req.prompt_ids)} tokens leaves no room "
                             f"under max_model_len {self.config.max_model_len}")
        self._check_fits(req)
        req.status = RequestStatus.WAITING
        self.waiting.append(req)

    def _check_fits(self, req: Request) -> None:
        """A prompt (and its first token) that no pool of the manager could ever hold is refused at the door."""
        for g, pool in enumerate(self.manager.pools):
            bs = self.manager.block_sizes[g]
            need = (len(req.prompt_ids) + 1 + bs - 1) // bs
            if need > pool.num_blocks:
                raise ValueError(f"request {req.req_id!r}: needs {need} pages, the pool has {pool.num_blocks}")

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, req_id: Hashable) -> Optional[Request]:
        for q in (self.running, self.waiting):
            for r in list(q):
                if r.req_id == req_id:
                    q.remove(r)
                    self._finish(r, FinishReason.ABORT)
                    return r
        return None

    # ---- one step's decisions
    def schedule(self, lookahead: bool = False) -> SchedulerOutput:
        cfg = self.config
        out = SchedulerOutput()
        budget = cfg.max_num_batched_tokens
        threshold = cfg.long_prefill_token_threshold
        i = 0
        max_len, exempt = cfg.max_model_len, cfg.decode_exempt_from_budget
        allocate = self.manager.allocate
        while i < len(self.running):
            req = self.running[i]
            ahead = req.num_placeholders
            n_out = len(req.output_ids)
            known = len(req.prompt_ids) + n_out + ahead         # tokens of the request, those in flight included
            computed = req.num_computed
            if ahead and (n_out + ahead >= req.params.max_tokens or known >= max_len):
                i += 1                          # the token in flight is its last: nothing more to run
                continue
            num_new = known - computed
            is_decode = num_new == 1 and computed > 0
            if threshold > 0:
                num_new = min(num_new, threshold)
            if not (is_decode and exempt):
                num_new = min(num_new, budget)
            if computed + num_new > max_len:
                num_new = max_len - computed
            if num_new <= 0:
                i += 1
                continue
            placed = True
            while not allocate(req.req_id, computed + num_new):
                victim = self.running[-1]
                if victim is req:
                    if len(self.running) > 1:
                        placed = False          # others run: sit this step out, keep the pages
                    else:
                        self.running.pop()      # alone and still no fit: it can never finish
                        self._finish(req, FinishReason.LENGTH)
                        out.finished.append(req)
                        placed = False
                    break
                self.running.pop()
                self._preempt(victim)
                out.preempted.append(victim)
            if not placed:
                if req.finished:
                    continue
                i += 1
                continue
            out.scheduled.append(ScheduledRequest(req, computed, num_new, computed + num_new == known, n_out + ahead))
            if not (is_decode and exempt):
                budget -= num_new
            i += 1

        if not out.preempted:
            while self.waiting and budget > 0 and len(self.running) < cfg.max_num_seqs:
                req = self.waiting[0]
                began = False
                if req.num_computed == 0 and self.manager.prefix_caching and req.req_id not in self.manager \
                        and req.params.prompt_logprobs is None:      # (those want every prompt position run)
                    # pages of an earlier request with the same beginning: those tokens are not run again
                    req.num_computed = self.manager.begin(req.req_id, req.tokens(0, req.num_tokens))
                    began = req.num_computed > 0
                num_new = req.num_tokens - req.num_computed
                if threshold > 0:
                    num_new = min(num_new, threshold)
                num_new = min(num_new, budget, cfg.max_model_len - req.num_computed)
                if num_new <= 0 or not self.manager.allocate(req.req_id, req.num_computed + num_new):
                    if began:
                        self.manager.free(req.req_id)
                        req.num_computed = 0
                    break
                self.waiting.popleft()
                req.status = RequestStatus.RUNNING
                self.running.append(req)
                out.scheduled.append(ScheduledRequest(req, req.num_computed, num_new,
                                                      req.num_computed + num_new == req.num_tokens,
                                                      len(req.output_ids)))
                budget -= num_new

        for s in out.scheduled:                 # the cache will hold these once the step has run
            s.request.num_computed += s.num_tokens
            if lookahead and s.samples:
                s.request.num_placeholders += 1
        return out

    def _preempt(self, req: Request) -> None:
        if req.req_id in self.manager:
            self.manager.free(req.req_id)
        req.num_computed = 0
        req.num_placeholders = 0                # a token in flight is still appended when it arrives (update)
        req.status = RequestStatus.WAITING
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)

    def _finish(self, req: Request, reason: FinishReason) -> None:
        req.status = RequestStatus.FINISHED
        req.finish_reason = reason
        if req.req_id in self.manager:
            self.manager.free(req.req_id)

    # ---- after the step
    def update(self, step: SchedulerOutput, sampled: Dict[Hashable, int]) -> List[Request]:
        """Append the sampled tokens, check the stop conditions, free what has finished."""
        done = []
        for s in step.scheduled:
            req = s.request
            if not s.samples or req.finished:
                continue                        # finished meanwhile: what a step ahead computed for it is dropped
            tok = int(sampled[req.req_id])
            req.output_ids.append(tok)
            reason = self._check_stop(req, tok)
            if req.status == RequestStatus.RUNNING:
                if req.num_placeholders > 0:
                    req.num_placeholders -= 1
                if reason is not None:
                    self.running.remove(req)
            elif reason is not None:            # preempted while this token was in flight, and it ends the request
                self.waiting.remove(req)
            if reason is not None:
                self._finish(req, reason)
                done.append(req)
        return done

    def _check_stop(self, req: Request, tok: int) -> Optional[FinishReason]:
        p = req.params
        n_out = len(req.output_ids)
        if n_out >= p.min_tokens:
            if not p.ignore_eos and tok in self.eos:
                return FinishReason.STOP
            if tok in p.stop_token_ids:
                return FinishReason.STOP
        if n_out >= p.max_tokens or req.num_tokens >= self.config.max_model_len:
            return FinishReason.LENGTH
        return None


class NativeScheduler(Scheduler):
    """The same scheduler with its decisions taken in C++ (``csrc/host_core.cpp``) over the C++ cache manager
    (``cache.native.NativeCacheManager``): pages, queues, preemption and the stop check all live there; this class
    keeps the ``Request`` objects of the Python interface in step with it.  ``schedule_columns`` / ``update_columns``
    are the same calls without the objects (columns in, columns out), for callers that keep no ``Request``."""

    _REASONS = {1: FinishReason.STOP, 2: FinishReason.LENGTH, 3: FinishReason.ABORT}

    def __init__(self, config: EngineConfig, manager, eos_token_ids: Sequence[int] = ()):
        import numpy as np
        from ctypes import c_int, c_int32, c_int64, c_longlong, c_void_p
        from ..cache.native import NativeCacheManager, library
        if not isinstance(manager, NativeCacheManager):
            raise TypeError("NativeScheduler works on a NativeCacheManager")
        super().__init__(config, manager, eos_token_ids)
        self._np = np
        lib = self._lib = library()
        P, I, L = c_void_p, c_int, c_int64
        for name, res, args in (("dh_sched_new", P, [P, I, I, I, I, I, P, I]), ("dh_sched_delete", None, [P]),
                                ("dh_sched_add", I, [P, L, P, I, I, I, I, P, I, I]), ("dh_sched_forget", None, [P, L]),
                                ("dh_sched_abort", I, [P, L]), ("dh_sched_counts", I, [P, P, P]),
                                ("dh_sched_queue", I, [P, I, P, I]), ("dh_sched_preemptions", c_longlong, [P]),
                                ("dh_sched_schedule", I, [P, I, I, P, P, P, P, P, P, P, P]),
                                ("dh_sched_update", I, [P, I, P, P, P, P, P])):
            f = getattr(lib, name)
            f.restype, f.argtypes = res, args
        eos = np.asarray(sorted(self.eos), dtype=np.int32)
        self._s = lib.dh_sched_new(manager._h, config.max_num_batched_tokens, config.long_prefill_token_threshold,
                                   config.max_model_len, config.max_num_seqs, int(config.decode_exempt_from_budget),
                                   eos.ctypes.data if eos.size else None, eos.size)
        self._reqs: Dict[int, Request] = {}                  # handle -> request, while the request lives
        cap = self._cap = max(16, 2 * config.max_num_seqs + 8)
        self._ids, self._pre, self._fin = (np.zeros(cap, dtype=np.int64) for _ in range(3))
        self._start, self._num, self._smp, self._gen = (np.zeros(cap, dtype=np.int32) for _ in range(4))
        self._counts = np.zeros(4, dtype=np.int32)
        self._tok, self._reason = np.zeros(cap, dtype=np.int32), np.zeros(cap, dtype=np.int32)
        self._done = np.zeros(cap, dtype=np.int64)

    def __del__(self):
        s, self._s = getattr(self, "_s", None), None
        if s:
            self._lib.dh_sched_delete(s)

    def _error(self) -> str:
        msg = self._lib.dh_last_error()
        return msg.decode("utf-8", "replace") if msg else "host core error"

    # ---- the queues as the Python scheduler shows them
    def _queue(self, which: int):
        np = self._np
        n = max(1, len(self._reqs))
        buf = np.zeros(n, dtype=np.int64)
        k = self._lib.dh_sched_queue(self._s, which, buf.ctypes.data, n)
        return [self._reqs[int(h)] for h in buf[:k]]

    @property
    def waiting(self):
        return deque(self._queue(0))

    @waiting.setter
    def waiting(self, value):            # (the base class's constructor sets empty queues)
        pass

    @property
    def running(self):
        return self._queue(1)

    @running.setter
    def running(self, value):
        pass

    @property
    def num_preemptions(self) -> int:
        return int(self._lib.dh_sched_preemptions(self._s)) if getattr(self, "_s", None) else 0

    @num_preemptions.setter
    def num_preemptions(self, value):
        pass

    def has_unfinished(self) -> bool:
        np = self._np
        w, r = np.zeros(1, dtype=np.int32), np.zeros(1, dtype=np.int32)
        self._lib.dh_sched_counts(self._s, w.ctypes.data, r.ctypes.data)
        return bool(w[0] or r[0])

    # ---- queue
    def add_request(self, req: Request) -> None:
        np = self._np
        req.params.validate()
        if not req.prompt_ids:
            raise ValueError(f"request {req.req_id!r}: empty prompt")
        if len(req.prompt_ids) >= self.config.max_model_len:
            raise ValueError(f"request {req.req_id!r}: prompt of {len(req.prompt_ids)} tokens leaves no room "
                             f"under max_model_len {self.config.max_model_len}")
        self._check_fits(req)
        h = self.manager.handle(req.req_id)
        prompt = np.ascontiguousarray(req.prompt_ids, dtype=np.int32)
        stops = np.ascontiguousarray(sorted(req.params.stop_token_ids), dtype=np.int32)
        p = req.params
        if self._lib.dh_sched_add(self._s, h, prompt.ctypes.data, prompt.size, int(min(p.max_tokens, 2 ** 31 - 1)),
                                  int(p.min_tokens), int(bool(p.ignore_eos)), stops.ctypes.data if stops.size else None,
                                  stops.size, int(p.prompt_logprobs is not None)):
            raise ValueError(self._error())
        req.status = RequestStatus.WAITING
        self._reqs[h] = req

    def _drop(self, h: int) -> None:
        req = self._reqs.pop(h, None)
        self._lib.dh_sched_forget(self._s, h)
        if req is not None:
            self.manager._forget_if_gone(req.req_id)

    def abort(self, req_id: Hashable) -> Optional[Request]:
        h = self.manager._ids.get(req_id)
        if h is None or h not in self._reqs or not self._lib.dh_sched_abort(self._s, h):
            return None
        req = self._reqs[h]
        req.status, req.finish_reason = RequestStatus.FINISHED, FinishReason.ABORT
        self._drop(h)
        return req

    # ---- one step's decisions
    def schedule_columns(self, lookahead: bool = False):
        """(handles, start, num_tokens, samples, num_generated, preempted handles, finished handles): views of
        buffers that the next call overwrites."""
        c = self._counts
        if self._lib.dh_sched_schedule(self._s, int(lookahead), self._cap, self._ids.ctypes.data, self._start.ctypes.data,
                                       self._num.ctypes.data, self._smp.ctypes.data, self._gen.ctypes.data,
                                       self._pre.ctypes.data, self._fin.ctypes.data, c.ctypes.data):
            raise RuntimeError(self._error())
        n, p, f = int(c[0]), int(c[1]), int(c[2])
        return (self._ids[:n], self._start[:n], self._num[:n], self._smp[:n], self._gen[:n], self._pre[:p], self._fin[:f])

    def schedule(self, lookahead: bool = False) -> SchedulerOutput:
        ids, start, num, smp, gen, pre, fin = self.schedule_columns(lookahead)
        out = SchedulerOutput()
        for h in pre.tolist():
            r = self._reqs[h]
            r.num_computed, r.num_placeholders, r.status = 0, 0, RequestStatus.WAITING
            r.num_preemptions += 1
            out.preempted.append(r)
        for h in fin.tolist():
            r = self._reqs[h]
            r.status, r.finish_reason = RequestStatus.FINISHED, FinishReason.LENGTH
            out.finished.append(r)
            self._drop(h)
        for h, s, n, m, g in zip(ids.tolist(), start.tolist(), num.tolist(), smp.tolist(), gen.tolist()):
            r = self._reqs[h]
            r.status = RequestStatus.RUNNING
            r.num_computed = s + n
            if lookahead and m:
                r.num_placeholders += 1
            out.scheduled.append(ScheduledRequest(r, s, n, bool(m), g))
        return out

    # ---- after the step
    def update_columns(self, handles, samples, tokens):
        """The sampled tokens of a step's scheduled requests (int32 columns as ``schedule_columns`` gave them, with
        the tokens); returns (handles that finished, reasons 1 = stop, 2 = length)."""
        n = len(handles)
        k = self._lib.dh_sched_update(self._s, n, handles.ctypes.data, samples.ctypes.data, tokens.ctypes.data,
                                      self._done.ctypes.data, self._reason.ctypes.data)
        return self._done[:k], self._reason[:k]

    def update(self, step: SchedulerOutput, sampled: Dict[Hashable, int]) -> List[Request]:
        np = self._np
        n = len(step.scheduled)
        ids = np.zeros(max(1, n), dtype=np.int64)
        smp = np.zeros(max(1, n), dtype=np.int32)
        tok = np.zeros(max(1, n), dtype=np.int32)
        for k, s in enumerate(step.scheduled):
            req = s.request
            ids[k] = self.manager._ids.get(req.req_id, -1) if not req.finished else -1
            if s.samples and not req.finished:
                smp[k], tok[k] = 1, int(sampled[req.req_id])
                req.output_ids.append(int(tok[k]))
                if req.status == RequestStatus.RUNNING and req.num_placeholders > 0:
                    req.num_placeholders -= 1
        done_h, reasons = self.update_columns(ids[:n], smp[:n], tok[:n])
        done = []
        for h, why in zip(done_h.tolist(), reasons.tolist()):
            req = self._reqs[h]
            req.status, req.finish_reason = RequestStatus.FINISHED, self._REASONS[why]
            done.append(req)
            self._drop(h)
        return done
