"""The packed plan of a step: the incremental plan of a decode graph equals the plan built from
scratch, step after step, under requests that come, go, are preempted and come back."""
import random

import numpy as np
import pytest
import torch

from dinfer_b200.cache.manager import CacheManager, GroupSpec
from dinfer_b200.engine.batch import DecodePlan, PlanBuilder, StepEntry


def packed(builder, entries, starts, bucket, width):
    dev = torch.zeros(builder.words(bucket, bucket, bucket, width), dtype=torch.int32)
    builder.build(entries, starts, pad_reqs=bucket, table_width=width, dev=dev)
    return dev.numpy().copy()


@pytest.mark.parametrize("groups", [[GroupSpec()], [GroupSpec(), GroupSpec(window=5)]])
def test_decode_plan_matches_full_build(groups):
    rng = random.Random(3)
    bs, width, bucket = 4, 12, 4
    m = CacheManager(groups, bs, 64, max_num_seqs=bucket)
    builder = PlanBuilder(m, "cpu", max_tokens=64, max_reqs=bucket, max_blocks=width)
    dev = torch.zeros(builder.words(bucket, bucket, bucket, width), dtype=torch.int32)
    plan = DecodePlan(builder, bucket, width, dev)
    live, next_id = {}, 0
    for step in range(300):
        # requests come (with some tokens already computed), go, or are preempted and readmitted
        if len(live) < bucket and rng.random() < 0.3:
            n0 = rng.randrange(1, 20)
            rid = f"r{next_id}"; next_id += 1
            assert m.allocate(rid, n0)
            m.advance(rid, n0)
            live[rid] = n0
        if live and rng.random() < 0.1:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        if live and rng.random() < 0.1:
            rid = rng.choice(list(live))
            n0 = live[rid]
            m.free(rid)
            assert m.allocate(rid, n0)
            m.advance(rid, n0)
        for rid in [r for r, n in live.items() if n + 1 > bs * width]:
            m.free(rid)
            del live[rid]
        order = list(live)
        rng.shuffle(order)
        entries = [StepEntry(r, [rng.randrange(100)], [0]) for r in order]
        starts = [live[r] for r in order]
        for e, s in zip(entries, starts):
            assert m.allocate(e.req_id, s + 1)
        want = packed(builder, entries, starts, bucket, width)
        plan.fill(entries, starts)
        got = dev.numpy()
        for name, (o, n) in plan.views.items():
            if name == "fresh":          # taken by whichever plan asks first
                continue
            assert np.array_equal(got[o:o + n], want[o:o + n]), f"step {step}: {name}"
        for e, s in zip(entries, starts):
            m.advance(e.req_id, s + 1)
            live[e.req_id] = s + 1
        m.check_invariants()
