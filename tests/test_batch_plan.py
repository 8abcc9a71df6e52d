"""The packed plan of a step: the incremental plan of a decode graph equals the plan built from
scratch, step after step, under requests that come, go, are preempted and come back."""
import random

import numpy as np
import pytest
import torch

from dinfer_b200.cache.manager import CacheManager, GroupSpec
from dinfer_b200.cache.native import NativeCacheManager
from dinfer_b200.engine.batch import DecodePlan, PlanBuilder, StepEntry


def packed(builder, entries, starts, bucket, width):
    dev = torch.zeros(builder.words(bucket, bucket, bucket, width), dtype=torch.int32)
    builder.build(entries, starts, pad_reqs=bucket, table_width=width, dev=dev)
    return dev.numpy().copy()


@pytest.mark.parametrize("manager", [CacheManager, NativeCacheManager])
@pytest.mark.parametrize("groups", [[GroupSpec()], [GroupSpec(), GroupSpec(window=5)],
                                    [GroupSpec(block_size=8), GroupSpec(window=5, block_size=2)]])
def test_decode_plan_matches_full_build(groups, manager):
    """(With the C++ cache manager the plan is written by the library from its own tables.)"""
    rng = random.Random(3)
    bs, width, bucket = 4, 12, 4
    m = manager(groups, bs, 64, max_num_seqs=bucket)
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
        for rid in [r for r, n in live.items() if n + 1 > min(m.block_sizes) * width]:
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


def test_which_steps_replay_a_graph():
    """The decision which steps with prompt portions have a shape that comes again (and is worth a captured graph):
    portions that fill the budget, few prompt tokens padded up to a power of two, and, for models small enough,
    more of them padded up to a multiple of 128 or 256."""
    from dinfer_b200.engine.runner import graph_shape
    buckets = [1, 2, 4, 8, 16]

    def shape(prompts, decodes=0, budget=2048, limit=128):
        return graph_shape(prompts, decodes, budget, buckets, (4, 16), 128, limit)

    assert shape([2048]) == (2048, 4, 0) and shape([1000, 1048], 5) == (2048, 4, 8)  # the budget, exactly
    assert shape([128] * 16) == (2048, 16, 0)                                        # many short prompts: more places
    assert shape([5]) == (16, 4, 0) and shape([16], 1) == (16, 4, 1) and shape([17, 3]) == (32, 4, 0)
    assert shape([100], 16) == (128, 4, 16) and shape([128]) == (128, 4, 0)
    assert shape([129]) is None and shape([2047]) is None                            # a large model: kernel by kernel
    assert shape([129], limit=4480) == (256, 4, 0) and shape([1025], limit=4480) == (1280, 4, 0)
    assert shape([2000], limit=4480) == (2048, 4, 0)                                 # never beyond the budget
    assert shape([600], limit=512) is None and shape([500], limit=512) == (512, 4, 0)
    assert shape([], 4) is None and shape([100], 17) is None                         # no portion; too many decodes
    assert shape([4, 4, 4, 4]) == (16, 4, 0)                                         # four portions, nothing to pad
    assert shape([4, 4, 4, 3]) == (16, 16, 0)                                        # the padding needs a fifth place
    assert shape([4] * 16) == (64, 16, 0)
    assert shape([4] * 15 + [3]) is None and shape([2] * 17) is None                 # 16 portions and padding; 17
    assert shape([40], budget=48) is None                                            # the padding would pass the budget
    assert shape([48], budget=48) == (48, 4, 0)


def test_dummy_places_of_a_captured_graph_stay_inside_the_tables_and_the_position_table():
    """A token budget above the longest request: the dummy portions a graph is captured on (and padded with) are
    spread over places no longer than that, or the step runs kernel by kernel; a plan whose dummy request is
    longer than its table covers, or whose positions leave the position table, does not pass the check."""
    from dinfer_b200.engine import batch as B
    from dinfer_b200.engine.runner import capture_places, graph_shape
    buckets, places = [1, 2, 4], (4, 16)
    # budget 512, longest request 96: a budget-filling step of 4 x 96 + 128 does not fit 4 or... it needs 16 places
    assert graph_shape([96, 96, 96, 96, 96, 32], 1, 512, buckets, places, 128, 10**6, longest=96) == (512, 16, 1)
    assert capture_places(512, 16, 1, 96) == [(-1, 96)] * 5 + [(-1, 32)] + [(-1, 0)] * 10 + [(-1, 1)]
    assert capture_places(512, 4, 0, 96) is None
    # 4 places of at most 96 cannot hold the 512 tokens of the capture: kernel by kernel
    assert graph_shape([96, 96, 64], 0, 256, buckets, (4,), 128, 10**6, longest=60) is None
    # a dummy portion longer than the longest request: kernel by kernel (130 tokens padded to 256 needs 126)
    assert graph_shape([70, 60], 0, 512, buckets, places, 128, 10**6, longest=100) is None
    assert graph_shape([70, 60], 0, 512, buckets, places, 128, 10**6, longest=128) == (256, 4, 0)
    assert graph_shape([70, 60], 0, 512, buckets, places, 128, 10**6) == (256, 4, 0)

    m = CacheManager([GroupSpec()], 4, 64, max_num_seqs=4)
    builder = PlanBuilder(m, "cpu", max_tokens=256, max_reqs=8, max_blocks=6, max_positions=24)
    old, B.VALIDATE_PLANS = B.VALIDATE_PLANS, True
    try:
        builder.build([], [], table_width=6, slots=capture_places(40, 4, 2, 24))          # 24 + 16 tokens: fine
        with pytest.raises(AssertionError, match="longer than its table"):
            builder.build([], [], table_width=6, slots=[(-1, 25), (-1, 1)])
        wide = PlanBuilder(m, "cpu", max_tokens=256, max_reqs=8, max_blocks=16, max_positions=24)
        with pytest.raises(AssertionError, match="position table"):
            wide.build([], [], table_width=16, slots=[(-1, 25), (-1, 1)])
    finally:
        B.VALIDATE_PLANS = old


def test_slots_and_tables_of_groups_with_page_sizes_of_their_own():
    """A token's slot in a group is page * (the group's page size) + offset, and every group's table is as wide as
    the plan says (the unused entries -1)."""
    m = CacheManager([GroupSpec(), GroupSpec(block_size=2)], 8, [16, 64], max_num_seqs=2)
    builder = PlanBuilder(m, "cpu", max_tokens=32, max_reqs=2, max_blocks=16)
    assert m.allocate("a", 13)
    ids, rows, ctx = builder.build([StepEntry("a", list(range(13)), [12])], [0])
    big, small = m.block_table("a", 0), m.block_table("a", 1)
    assert (len(big), len(small)) == (2, 7)
    g0, g1 = ctx.groups
    assert (g0.block_size, g1.block_size) == (8, 2)
    assert g0.block_table.shape == g1.block_table.shape == (1, 7)              # one width: what the small pages need
    assert g0.block_table[0].tolist() == big + [-1] * 5 and g1.block_table[0].tolist() == small
    assert g0.slot_mapping.tolist() == [big[p // 8] * 8 + p % 8 for p in range(13)]
    assert g1.slot_mapping.tolist() == [small[p // 2] * 2 + p % 2 for p in range(13)]


def test_pair_bound_of_the_prompt_attention_holds_for_every_spread_of_the_tokens():
    """A graph is captured with all prompt tokens in one place and replayed with them spread over the places: the
    bound made at capture covers every such spread, and requests with one token add nothing."""
    import random
    from dinfer_b200.kernels.attention_ops import umma_pair_bound
    rng = random.Random(5)
    for _ in range(300):
        group = rng.choice([1, 2, 4, 8, 16])
        places = rng.choice([1, 4, 16])
        total = rng.randint(2, 3000)
        decodes = [1] * rng.randint(0, 70)
        bound = umma_pair_bound([total] + [0] * (places - 1) + decodes, group)
        cuts = sorted(rng.randint(0, total) for _ in range(places - 1))
        lens = [b - a for a, b in zip([0] + cuts, cuts + [total])]
        pairs = sum((n * group + 255) // 256 for n in lens if n > 1)
        assert pairs <= bound <= (total * group) // 256 + places, (lens, group, bound)


def test_the_longest_prompt_request_of_a_step_is_told_apart_from_the_longest_request():
    """``max_prefill_seq_len`` counts only requests that bring more than one token: a short new prompt beside a
    long decoding request still counts as a short context for the parts that choose by it."""
    m = CacheManager([GroupSpec()], 8, [64], max_num_seqs=4)
    builder = PlanBuilder(m, "cpu", max_tokens=64, max_reqs=4, max_blocks=32)
    assert m.allocate("old", 200) and m.allocate("new", 9) and m.allocate("more", 40)
    m.advance("old", 199)
    m.advance("more", 30)
    entries = [StepEntry("old", [5], [0]), StepEntry("new", list(range(9)), [8]), StepEntry("more", list(range(10)), [])]
    ids, rows, ctx = builder.build(entries, [199, 0, 30])
    assert ctx.max_seq_len == 200 and ctx.max_prefill_seq_len == 40 and ctx.max_q_len == 10
    ids, rows, ctx = builder.build(entries[:1], [199])
    assert ctx.max_prefill_seq_len == 0 and ctx.all_decode
