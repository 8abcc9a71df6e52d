"""The scheduler's decisions, driven with a fake step function that returns f(sequence length)
in the manner of the reference's Echo executor (crates/core/src/runner.rs:888-905).  No GPU."""
import pytest

import sys

from dinfer_b200.cache.manager import CacheManager, GroupSpec
from dinfer_b200.cache.native import NativeCacheManager
from dinfer_b200.config.engine_config import EngineConfig
from dinfer_b200.engine.request import FinishReason, Request, RequestStatus
from dinfer_b200.engine.scheduler import NativeScheduler, Scheduler
from dinfer_b200.sampling.params import SamplingParams


@pytest.fixture(params=["python", "native"], autouse=True)
def implementation(request, monkeypatch):
    """Every test of this file runs twice: on the Python scheduler and cache manager, and on the C++ ones."""
    if request.param == "native":
        monkeypatch.setattr(sys.modules[__name__], "CacheManager", NativeCacheManager)
        monkeypatch.setattr(sys.modules[__name__], "Scheduler", NativeScheduler)
    return request.param



def make(num_blocks=64, block_size=4, **kw):
    cfg = EngineConfig(block_size=block_size, num_blocks=num_blocks,
                       **{"max_model_len": 64, "max_num_seqs": 4, "max_num_batched_tokens": 16, **kw})
    m = CacheManager([GroupSpec()], block_size, num_blocks, cfg.max_num_seqs,
                     enable_prefix_caching=cfg.enable_prefix_caching)
    return Scheduler(cfg, m, eos_token_ids=[99]), m


def req(i, n, **p):
    return Request(i, list(range(1, n + 1)), SamplingParams(**{"max_tokens": 8, "temperature": 0.0, **p}), seed=1)


def run_step(s, m, token=lambda r: 1000 + r.num_tokens):
    out = s.schedule()
    for x in out.scheduled:                       # what the step function does to the cache
        assert x.request.req_id in m and m.num_tokens(x.request.req_id) >= x.start + x.num_tokens
        assert m.num_computed(x.request.req_id) == x.start
        m.advance(x.request.req_id, x.start + x.num_tokens,
                  x.request.tokens(x.start, x.start + x.num_tokens) if m.prefix_caching else None)
    done = s.update(out, {x.request.req_id: token(x.request) for x in out.scheduled if x.samples})
    m.check_invariants()
    return out, done


def test_prompt_is_cut_by_the_budget_then_decodes():
    s, m = make()
    r = req("a", 40)
    s.add_request(r)
    sizes = []
    for _ in range(3):
        out, _ = run_step(s, m)
        sizes.append([(x.start, x.num_tokens, x.samples) for x in out.scheduled])
    assert sizes == [[(0, 16, False)], [(16, 16, False)], [(32, 8, True)]]
    assert r.output_ids == [1040]
    out, _ = run_step(s, m)
    assert [(x.start, x.num_tokens, x.samples) for x in out.scheduled] == [(40, 1, True)]


def test_first_come_first_served_shares_the_budget():
    s, m = make()
    s.add_request(req("a", 10))
    s.add_request(req("b", 10))
    s.add_request(req("c", 3))
    out, _ = run_step(s, m)
    assert [(x.request.req_id, x.num_tokens) for x in out.scheduled] == [("a", 10), ("b", 6)]
    out, _ = run_step(s, m)      # a decodes (exempt from the budget), b's rest, then c
    assert [(x.request.req_id, x.start, x.num_tokens) for x in out.scheduled] == [("a", 10, 1), ("b", 6, 4), ("c", 0, 3)]


def test_decode_counts_against_budget_when_not_exempt():
    s, m = make(decode_exempt_from_budget=False, max_num_batched_tokens=4)
    for i in range(3):
        s.add_request(req(i, 2))
    run_step(s, m)                # 0 and 1 prefill (2+2)
    out, _ = run_step(s, m)       # two decodes take 2 of the 4 tokens, request 2 gets the other 2
    assert [(x.request.req_id, x.num_tokens) for x in out.scheduled] == [(0, 1), (1, 1), (2, 2)]


def test_max_num_seqs_and_long_prefill_threshold():
    s, m = make(max_num_seqs=2, long_prefill_token_threshold=5)
    for i in range(3):
        s.add_request(req(i, 12))
    out, _ = run_step(s, m)
    assert [(x.request.req_id, x.num_tokens) for x in out.scheduled] == [(0, 5), (1, 5)]
    assert len(s.waiting) == 1


def test_stop_conditions():
    s, m = make()
    a, b, c, d, e = req("a", 3), req("b", 3, ignore_eos=True, max_tokens=3), req("c", 3, stop_token_ids=[5]), \
        req("d", 3, min_tokens=2), req("e", 3)
    for r in (a, b, c, d):
        s.add_request(r)
    tok = {"a": [99], "b": [99, 99, 99], "c": [7, 5], "d": [99, 99]}
    n = {k: 0 for k in tok}

    def token(r):
        n[r.req_id] += 1
        return tok[r.req_id][n[r.req_id] - 1]
    for _ in range(4):
        run_step(s, m, token)
    assert (a.finish_reason, a.output_ids) == (FinishReason.STOP, [99])
    assert (b.finish_reason, b.output_ids) == (FinishReason.LENGTH, [99, 99, 99])
    assert (c.finish_reason, c.output_ids) == (FinishReason.STOP, [7, 5])
    assert (d.finish_reason, d.output_ids) == (FinishReason.STOP, [99, 99])     # the first eos came too early
    assert not s.has_unfinished() and m.num_free_blocks() == 64
    s2, m2 = make(max_model_len=6)
    s2.add_request(e)
    for _ in range(5):
        run_step(s2, m2)
    assert e.finish_reason == FinishReason.LENGTH and e.num_tokens == 6


def test_out_of_pages_preempts_the_last_and_recomputes():
    s, m = make(num_blocks=6, block_size=4)        # 24 tokens of cache in all
    a, b = req("a", 8, max_tokens=20), req("b", 8, max_tokens=20)
    s.add_request(a)
    s.add_request(b)
    run_step(s, m)                                 # both prompts: 2 + 2 pages
    assert m.num_free_blocks() == 2
    for _ in range(4):
        run_step(s, m)                             # each takes a third page, then fills it
    assert m.num_free_blocks() == 0 and a.num_tokens == 13 and a.num_computed == 12
    out, _ = run_step(s, m)                        # a needs a 4th page: b, the last one, is preempted
    assert [r.req_id for r in out.preempted] == ["b"] and [x.request.req_id for x in out.scheduled] == ["a"]
    assert b.status == RequestStatus.WAITING and b.num_computed == 0 and s.waiting[0] is b
    assert "b" not in m and b.num_preemptions == 1 and len(b.output_ids) == 5      # its tokens are kept
    kept = list(b.output_ids)
    steps = 0
    while s.has_unfinished() and steps < 200:
        out, _ = run_step(s, m)
        steps += 1
        if any(x.request is b for x in out.scheduled) and b.num_preemptions == 1 and b.output_ids[:5] == kept:
            first = [x for x in out.scheduled if x.request is b][0]
            if first.start == 0:
                assert first.num_tokens == 8 + 5     # recomputed from token 0, its own outputs included
    assert a.finished and b.finished and m.num_free_blocks() == 6
    assert len(a.output_ids) == 20 - 0 or a.finish_reason == FinishReason.LENGTH


def test_nothing_admitted_in_a_step_that_preempted():
    s, m = make(num_blocks=4, block_size=4)
    a, b, c = req("a", 8), req("b", 8), req("c", 2)
    s.add_request(a)
    s.add_request(b)
    run_step(s, m)
    s.add_request(c)
    out, _ = run_step(s, m)            # a's 9th token needs a page: b goes; c must wait although it would fit
    assert [r.req_id for r in out.preempted] == ["b"]
    assert [x.request.req_id for x in out.scheduled] == ["a"]
    assert [r.req_id for r in s.waiting] == ["b", "c"]


def test_sole_request_that_cannot_fit_ends_with_length():
    s, m = make(num_blocks=3, block_size=4)
    a = req("a", 10, max_tokens=30)
    s.add_request(a)
    done = []
    for _ in range(10):
        out, d = run_step(s, m)
        done += out.finished + d
        if a.finished:
            break
    assert a.finish_reason == FinishReason.LENGTH and a.num_tokens == 13     # 12 cached + the last sampled
    assert m.num_free_blocks() == 3 and not s.has_unfinished()


def test_refused_at_the_door():
    s, m = make(num_blocks=3, block_size=4)
    with pytest.raises(ValueError, match="pages"):
        s.add_request(req("big", 20))
    with pytest.raises(ValueError, match="max_model_len"):
        s.add_request(req("long", 64))
    with pytest.raises(ValueError, match="empty"):
        s.add_request(Request("e", [], SamplingParams()))
    with pytest.raises(ValueError, match="top_p"):
        s.add_request(req("p", 3, top_p=0.0))


def test_abort_frees_pages():
    s, m = make()
    a = req("a", 9)
    s.add_request(a)
    run_step(s, m)
    assert m.num_free_blocks() < 64
    s.abort("a")
    assert a.finish_reason == FinishReason.ABORT and m.num_free_blocks() == 64 and not s.has_unfinished()


def test_prefix_cache_skips_the_tokens_an_earlier_request_left():
    s, m = make(enable_prefix_caching=True)
    s.add_request(req("a", 14, max_tokens=2))
    while s.has_unfinished():
        run_step(s, m)
    # the same 14 prompt tokens: 3 whole pages of 4 are found, the rest is run
    s.add_request(req("b", 14, max_tokens=2))
    out, _ = run_step(s, m)
    assert [(x.request.req_id, x.start, x.num_tokens, x.samples) for x in out.scheduled] == [("b", 12, 2, True)]
    assert m.prefix_hits == 12
    # a request that is preempted finds its own pages again when it comes back
    s2, m2 = make(num_blocks=9, enable_prefix_caching=True, max_num_batched_tokens=32)
    s2.add_request(req("x", 16, max_tokens=30))
    s2.add_request(req("y", 16, max_tokens=30))
    preempted = False
    for _ in range(60):
        out, _ = run_step(s2, m2)
        preempted |= bool(out.preempted)
        if not s2.has_unfinished():
            break
    assert preempted and not s2.has_unfinished()
    assert m2.prefix_hits > 0


# ---- scheduling one step ahead (the tokens of a step are read after the next one is scheduled)
def drive(s, m, ahead, token, max_steps=400):
    """Run until nothing is left, the way the engine loop does: with ``ahead`` the next step is scheduled and
    its cache bookkeeping done BEFORE the last step's tokens are applied.  ``token(req, length)`` is the token a
    step yields for a request whose sequence is ``length`` long after the step (a pure function, so both ways
    of driving must generate the same sequences)."""
    plans, flight, steps = [], None, 0

    def collect(f):
        plan, toks, ahead_of = f
        done = s.update(plan, toks)
        for rid in ahead_of:                        # tokens the next step took without knowing them
            if rid in m:
                m.resolve(rid, [toks[rid]])
        return done

    while (s.has_unfinished() or flight is not None) and steps < max_steps:
        steps += 1
        plan = s.schedule(lookahead=ahead)
        toks = {}
        for x in plan.scheduled:
            r = x.request
            end = x.start + x.num_tokens
            assert r.req_id in m and m.num_tokens(r.req_id) >= end
            assert m.num_computed(r.req_id) == x.start
            assert end <= r.num_tokens + 1                              # at most one token not yet read
            ids = r.tokens(x.start, min(end, r.num_tokens))
            if end > r.num_tokens:
                ids = ids + [-1]
                flight[2].add(r.req_id)
            m.advance(r.req_id, end, ids if m.prefix_caching else None)
            if x.samples:
                toks[r.req_id] = token(r, end)
        plans.append(plan)
        if flight is not None:
            collect(flight)
            flight = None
        if plan.scheduled:
            flight = (plan, toks, set())
            if not ahead:
                collect(flight)
                flight = None
        m.check_invariants()
    assert steps < max_steps
    return plans


@pytest.mark.parametrize("num_blocks", [64, 7])
def test_scheduling_ahead_generates_the_same_sequences(num_blocks):
    """Prompts in portions, decoding, an end-of-sequence token, max_tokens, and (with 7 pages) preemption with a
    token in flight: the sequences do not depend on whether the host reads tokens at once or a step late."""
    def token(r, length):
        return 99 if (r.req_id == "b" and length == 14) else 1000 + length

    results = {}
    for ahead in (False, True):
        s, m = make(num_blocks=num_blocks, block_size=4, max_num_batched_tokens=8)
        reqs = [req("a", 9, max_tokens=12), req("b", 10, max_tokens=12), req("c", 3, max_tokens=5)]
        for r in reqs:
            s.add_request(r)
        plans = drive(s, m, ahead, token)
        assert all(r.finished for r in reqs) and m.num_free_blocks() == num_blocks
        results[ahead] = [(r.req_id, list(r.output_ids), r.finish_reason) for r in reqs]
        if ahead:
            assert all(r.num_placeholders == 0 for r in reqs if r.finish_reason == FinishReason.LENGTH)
        if num_blocks == 7:
            assert s.num_preemptions > 0
    assert results[False] == results[True]
    b = results[True][1]
    assert b[1][-1] == 99 and b[2] == FinishReason.STOP and len(b[1]) == 5


def test_scheduling_ahead_does_not_run_past_a_certain_end():
    """max_tokens is known before the token arrives: the request is not scheduled for a step that cannot count;
    an end-of-sequence token is not: one step runs in vain and its token is dropped."""
    s, m = make()
    a = req("a", 4, max_tokens=3)
    s.add_request(a)
    plans = drive(s, m, True, lambda r, n: 1000 + n)
    assert [len(p.scheduled) for p in plans] == [1, 1, 1, 0]          # 3 tokens, then only the last read
    assert a.output_ids == [1004, 1005, 1006] and a.finish_reason == FinishReason.LENGTH
    s, m = make()
    b = req("b", 4, max_tokens=8)
    s.add_request(b)
    plans = drive(s, m, True, lambda r, n: 99 if n == 5 else 1000 + n)
    assert b.output_ids == [1004, 99] and b.finish_reason == FinishReason.STOP
    assert [len(p.scheduled) for p in plans] == [1, 1, 1, 0]          # the third ran before the 99 was read
    assert m.num_free_blocks() == 64


def test_scheduling_ahead_with_the_prefix_cache():
    """Tokens that a step took without knowing them reach the cache manager when they are read (``resolve``): the
    pages they fill become findable, later requests with the same beginning skip them, and the sequences are
    those of one step at a time."""
    results = {}
    for ahead in (False, True):
        s, m = make(num_blocks=40, block_size=4, max_num_batched_tokens=8, enable_prefix_caching=True)
        first = req("a", 9, max_tokens=12)
        s.add_request(first)
        drive(s, m, ahead, lambda r, n: 1000 + n)
        assert first.finished and m.num_free_blocks() == 40
        # the second request repeats the first one's prompt and its first outputs
        again = Request("b", first.prompt_ids + first.output_ids[:7] + [5, 6], SamplingParams(max_tokens=4, temperature=0.0), seed=1)
        s.add_request(again)
        plans = drive(s, m, ahead, lambda r, n: 1000 + n)
        first_run = [x for p in plans for x in p.scheduled if x.request is again][0]
        assert first_run.start == 16                 # four full pages of prompt and generated tokens were found
        results[ahead] = (list(first.output_ids), list(again.output_ids), m.prefix_hits)
        m.check_invariants()
    assert results[False] == results[True]
