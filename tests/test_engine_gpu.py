"""The engine through its Python entry point: greedy and sampled generation against the plain
implementation, long decoding, the first tokens, preemption under a small pool, and the
workloads set for the two tiny configurations."""
import random

import pytest
import torch

import helpers as H
import plain_model as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for name in ("A", "B"):
        d = tmp_path_factory.mktemp(f"gen{name}")
        out[name] = H.make_model_dir(str(d), H.CONFIGS[name], *H.INIT[name], torch.float32)
    return out


def plain_sampled(W, cfg, prompt, n, temperature, seed, **kw):
    seq, out = list(prompt), []
    for i in range(n):
        logits = P.qwen3_logits(W, cfg, seq)[-1]
        tok = P.sample_token(logits, temperature, seed, i, **kw)
        out.append(tok)
        seq.append(tok)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_tiny_a(dirs, dtype):
    """Tiny A's workload: prompts of 1, 7 and 19 tokens, greedy, 12 tokens each, pages of 4 tokens."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_A
    rng = random.Random(0)
    prompts = [H.random_tokens(rng, n, cfg["vocab_size"]) for n in (1, 7, 19)]
    W = H.load_plain_weights(dirs["A"])
    llm = LLM(dirs["A"], dtype=dtype, max_model_len=64, max_num_seqs=4, max_num_batched_tokens=16,
              num_blocks=40, block_size=4, enable_cuda_graph=False)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        want = P.greedy_generate(W, cfg, p, 12)
        assert o.finish_reason == "length" and len(o.output_ids) == 12
        if dtype == "float32":
            assert o.output_ids == want
        else:   # bfloat16 may leave the path at a near-tie; up to there the tokens are the same
            same = sum(1 for a, b in zip(o.output_ids, want) if a == b)
            first_diff = next((i for i, (a, b) in enumerate(zip(o.output_ids, want)) if a != b), 12)
            if first_diff < 12:
                lg = P.qwen3_logits(W, cfg, p + want[:first_diff])[-1]
                top = torch.topk(lg, 2).values
                assert float(top[0] - top[1]) < 0.05 * float(lg.abs().max()), (first_diff, same)
    assert llm.runner.manager.num_free_blocks() == 40


def test_sampled_generation_tiny_b(dirs):
    """Tiny B's workload: prompts of 3, 16, 17, 40, 63 tokens, portions of 8 mixed with decodes,
    20 tokens each at temperature 0.8 with sampling seed 7; 32-bit so that the draws are the same."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_B
    rng = random.Random(1)
    prompts = [H.random_tokens(rng, n, cfg["vocab_size"]) for n in (3, 16, 17, 40, 63)]
    W = H.load_plain_weights(dirs["B"])
    llm = LLM(dirs["B"], dtype="float32", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=8,
              num_blocks=24, block_size=16, enable_cuda_graph=False)
    sp = SamplingParams(temperature=0.8, seed=7, max_tokens=20, ignore_eos=True)
    outs = llm.generate(prompts, sp)
    agree = 0
    for p, o in zip(prompts, outs):
        want = plain_sampled(W, cfg, p, 20, 0.8, 7)
        assert len(o.output_ids) == 20
        agree += o.output_ids == want
    assert agree >= 4          # a draw within rounding of a boundary may differ in at most one request
    assert llm.runner.manager.num_free_blocks() == 24
    # the same request gives the same tokens alone and with top-k / top-p set
    solo = llm.generate([prompts[2]], sp)[0].output_ids
    assert solo == outs[2].output_ids
    sp2 = SamplingParams(temperature=1.0, seed=3, max_tokens=10, top_k=5, top_p=0.9, ignore_eos=True)
    got = llm.generate([prompts[1]], sp2)[0].output_ids
    assert got == plain_sampled(W, cfg, prompts[1], 10, 1.0, 3, top_k=5, top_p=0.9)


def test_preemption_gives_the_same_tokens(dirs):
    """A pool too small for all requests at once: some are preempted and recomputed; every request
    still gets the tokens it gets alone."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_B
    rng = random.Random(5)
    prompts = [H.random_tokens(rng, n, cfg["vocab_size"]) for n in (30, 28, 33, 25)]
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    big = LLM(dirs["B"], dtype="float32", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32,
              num_blocks=128, block_size=4, enable_cuda_graph=False)
    want = [o.output_ids for o in big.generate(prompts, sp)]
    assert big.stats.preemptions == 0
    del big
    small = LLM(dirs["B"], dtype="float32", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32,
                num_blocks=40, block_size=4, enable_cuda_graph=False)        # 160 tokens for 4 x ~70
    outs = small.generate(prompts, sp)
    assert small.stats.preemptions > 0
    assert [o.output_ids for o in outs] == want
    assert small.runner.manager.num_free_blocks() == 40
    small.runner.manager.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuda_graph_decode_equals_eager(dirs, dtype):
    """Decode-only steps replayed from a captured graph (batch padded to the bucket) give the logits
    of the eager path; requests join and leave so that several buckets and dummy rows are used."""
    from dinfer_b200.config.engine_config import EngineConfig
    from dinfer_b200.engine.batch import StepEntry
    from dinfer_b200.engine.runner import ModelRunner
    cfg = H.TINY_B
    rng = random.Random(11)
    toks = {r: H.random_tokens(rng, n, cfg["vocab_size"]) for r, n in {"a": 40, "b": 23, "c": 31, "d": 18, "e": 9}.items()}
    oracle = H.PlainOracle(dirs["B"])
    runs = {}
    for graphs in (False, True):
        r = ModelRunner.from_dir(dirs["B"], EngineConfig(max_model_len=64, max_num_seqs=6, max_num_batched_tokens=64,
                                                         num_blocks=40, block_size=4, dtype=dtype,
                                                         enable_cuda_graph=graphs))
        got = {k: [] for k in toks}
        # prompts of 5 tokens each in one mixed step, then token by token, requests dropping out as they end
        out = r.step([StepEntry(k, t[:5], [4]) for k, t in toks.items()])
        for i, k in enumerate(toks):
            got[k].append(out[i].cpu())
        p = 5
        while any(len(t) > p for t in toks.values()):
            live = [k for k, t in toks.items() if len(t) > p]
            out = r.step([StepEntry(k, [toks[k][p]], [0] if (p % 3 or k != "a") else []) for k in live])
            j = 0
            for k in live:
                if p % 3 or k != "a":
                    got[k].append(out[j].cpu())
                    j += 1
            for k in live:
                if len(toks[k]) == p + 1:
                    r.finish(k)
            p += 1
        assert r.manager.num_free_blocks() == 40
        if graphs:
            assert sorted(r._graphs) == [1, 2, 4, 6]
        runs[graphs] = got
    for k, t in toks.items():
        want = oracle.logits(t)
        rows = [4] + [q for q in range(5, len(t)) if (q % 3 or k != "a")]
        g = torch.stack(runs[True][k]).numpy()
        e = torch.stack(runs[False][k]).numpy()
        assert H.rel_err(g, want[rows]) <= H.TOLERANCE[dtype]
        assert H.rel_err(e, want[rows]) <= H.TOLERANCE[dtype]
        if dtype == "float32":
            assert (g == e).all()


def test_stop_token_and_eos(dirs):
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_A
    W = H.load_plain_weights(dirs["A"])
    prompt = [9, 8, 7, 6]
    path = P.greedy_generate(W, cfg, prompt, 10)
    llm = LLM(dirs["A"], dtype="float32", max_model_len=64, max_num_seqs=2, max_num_batched_tokens=16,
              num_blocks=32, block_size=4, enable_cuda_graph=False)
    o = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=10, stop_token_ids=[path[3]],
                                              ignore_eos=True))[0]
    cut = path.index(path[3]) + 1
    assert o.output_ids == path[:cut] and o.finish_reason == "stop"


def test_long_decoding_and_first_tokens(dirs):
    """Decode one token at a time up to the model's longest sequence; every position's logits are
    compared, the first ones included."""
    from dinfer_b200.config.engine_config import EngineConfig
    from dinfer_b200.engine.batch import StepEntry
    from dinfer_b200.engine.runner import ModelRunner
    cfg = H.TINY_B
    ids = H.random_tokens(random.Random(3), 256, cfg["vocab_size"])
    want = H.PlainOracle(dirs["B"]).logits(ids)
    for dtype in ("float32", "bfloat16"):
        r = ModelRunner.from_dir(dirs["B"], EngineConfig(max_model_len=256, max_num_seqs=2,
                                                         max_num_batched_tokens=64, num_blocks=17, block_size=16,
                                                         dtype=dtype, enable_cuda_graph=False))
        got = torch.cat([r.step([StepEntry("x", [t], [0])]) for t in ids]).cpu().numpy()
        r.finish("x")
        assert H.rel_err(got, want) <= H.TOLERANCE[dtype], dtype
        assert H.rel_err(got[:4], want[:4]) <= H.TOLERANCE[dtype]
        with pytest.raises(ValueError, match="max_model_len"):
            r.step([StepEntry("y", ids + [1], [])])
        with pytest.raises(ValueError, match="vocabulary"):
            r.step([StepEntry("z", [cfg["vocab_size"]], [0])])


def test_out_of_pages_is_an_error_at_the_step_function(dirs):
    from dinfer_b200.config.engine_config import EngineConfig
    from dinfer_b200.engine.batch import OutOfPages, StepEntry
    from dinfer_b200.engine.runner import ModelRunner
    r = ModelRunner.from_dir(dirs["A"], EngineConfig(max_model_len=64, max_num_seqs=4, max_num_batched_tokens=64,
                                                     num_blocks=4, block_size=4, dtype="float32",
                                                     enable_cuda_graph=False))
    r.step([StepEntry("a", list(range(12)), [])])
    with pytest.raises(OutOfPages):
        r.step([StepEntry("b", list(range(8)), [])])
    # a step whose LATER entry does not fit changes nothing for the earlier ones either
    free, slots = r.manager.num_free_blocks(), r.manager.state_slots.num_free
    with pytest.raises(OutOfPages):
        r.step([StepEntry("a", [1], []), StepEntry("c", [1, 2, 3], []), StepEntry("d", list(range(8)), [])])
    assert r.manager.num_free_blocks() == free and r.manager.state_slots.num_free == slots
    assert r.manager.requests() == ["a"] and r.manager.num_tokens("a") == 12 and r.manager.num_computed("a") == 12
    r.manager.check_invariants()
    r.finish("a")
    assert r.step([StepEntry("b", list(range(8)), [7])]).shape == (1, 256)


def test_prefix_caching_gives_the_same_tokens_and_skips_the_shared_beginning(dirs):
    """Requests that begin alike, one after the other and all at once, with the prefix cache on: the
    tokens of the plain implementation, fewer prompt tokens run, pages shared and given back."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_B
    rng = random.Random(21)
    stem = H.random_tokens(rng, 45, cfg["vocab_size"])
    prompts = [stem + H.random_tokens(rng, n, cfg["vocab_size"]) for n in (3, 11, 0, 20)] + [stem[:30]]
    prompts[2] = list(prompts[0])                            # an exact repeat
    W = H.load_plain_weights(dirs["B"])
    want = [P.greedy_generate(W, cfg, p, 6) for p in prompts]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    llm = LLM(dirs["B"], dtype="float32", max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32,
              num_blocks=64, block_size=8, enable_prefix_caching=True)
    got = [llm.generate([p], sp)[0].output_ids for p in prompts]          # one after the other: later ones hit
    assert got == want
    # the stem's five whole pages (40 tokens) for three followers, 24 of the 30-token prompt for the last
    assert llm.stats.prefix_hit_tokens >= 3 * 40 + 24
    ran = llm.stats.prompt_tokens
    assert ran == sum(len(p) for p in prompts) - llm.stats.prefix_hit_tokens
    llm.runner.manager.check_invariants()
    assert llm.runner.manager.num_free_blocks() == 64
    got2 = [o.output_ids for o in llm.generate(prompts, sp)]             # all at once, chunked and mixed
    assert got2 == want
    llm.runner.manager.check_invariants()
    assert llm.runner.manager.num_free_blocks() == 64


@pytest.mark.parametrize("prefix", [False, True])
def test_many_requests_small_pool_all_options(tmp_path, prefix):
    """A busy engine on the tensor-core head geometry (head size 128, groups of 4), bfloat16, CUDA graphs,
    a pool small enough to preempt, every sampling option, with and without the prefix cache: everything
    finishes within its limits, the books balance, no kernel gave up a wait, the greedy requests get the plain
    implementation's tokens (up to near-ties), and a second run with the same seeds gives the same tokens."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_D
    d = H.make_model_dir(str(tmp_path / "d"), cfg, *H.INIT["D"], torch.bfloat16)
    oracle = H.PlainOracle(d)

    def run():
        rng = random.Random(5)
        llm = LLM(d, dtype="bfloat16", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=96,
                  num_blocks=36, block_size=16, enable_prefix_caching=prefix)
        stem = H.random_tokens(rng, 70, cfg["vocab_size"])
        prompts, params = [], []
        for i in range(24):
            n = rng.choice([1, 2, 15, 16, 17, 60, 130, 200])
            p = (stem[:rng.choice([32, 48, 70])] if i % 3 == 0 else []) + H.random_tokens(rng, n, cfg["vocab_size"])
            prompts.append(p)
            kind = i % 4
            params.append(SamplingParams(
                temperature=[0.0, 0.8, 1.0, 0.6][kind], top_k=[-1, -1, 20, 50][kind], top_p=[1.0, 1.0, 0.9, 0.95][kind],
                min_p=0.02 if kind == 3 else 0.0, repetition_penalty=1.1 if kind == 2 else 1.0,
                max_tokens=rng.choice([1, 5, 40, 90]), seed=1000 + i, ignore_eos=(i % 5 != 0)))
        outs = llm.generate(prompts, params)
        llm.runner.check_device_status()
        llm.runner.manager.check_invariants()
        assert llm.runner.manager.num_free_blocks() == 36
        for o, sp, p in zip(outs, params, prompts):
            assert 1 <= len(o.output_ids) <= sp.max_tokens
            assert all(0 <= t < cfg["vocab_size"] for t in o.output_ids)
            if o.finish_reason == "length":
                assert len(o.output_ids) == sp.max_tokens or len(p) + len(o.output_ids) >= 512
        # the greedy requests (no penalty, no filter): the plain implementation's tokens, up to near-ties
        greedy = [(p, o) for p, o, sp in zip(prompts, outs, params) if sp.temperature == 0.0]
        assert len(greedy) >= 5
        exact = sum(H.check_greedy(oracle, p, o.output_ids) for p, o in greedy)
        assert exact >= 0.9 * sum(len(o.output_ids) for _, o in greedy)
        return [o.output_ids for o in outs], llm.stats

    first, stats = run()
    second, _ = run()
    assert first == second
    assert stats.preemptions > 0
    if prefix:
        assert stats.prefix_hit_tokens > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scheduling_ahead_gives_the_same_tokens(dirs, tmp_path, dtype):
    """One step kept in flight (the host reads a step's tokens after it has launched the next, which takes
    them on the device) against one step at a time: prompts in portions beside decoding requests, stop tokens
    (so that steps run in vain and are dropped), max_tokens, a pool small enough to preempt requests whose
    token is in flight, greedy and seeded sampling.  In 32-bit the tokens must be the same; in bfloat16
    (where a batch of another size may round differently) everything must finish within its limits."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_B if dtype == "float32" else H.TINY_D
    d = dirs["B"] if dtype == "float32" else H.make_model_dir(str(tmp_path / "d"), cfg, *H.INIT["D"], torch.bfloat16)
    stops = list(range(0, cfg["vocab_size"], 40))
    oracle = H.PlainOracle(d)

    def run(ahead):
        rng = random.Random(11)
        llm = LLM(d, dtype=dtype, max_model_len=256, max_num_seqs=6, max_num_batched_tokens=48,
                  num_blocks=13, block_size=16, async_scheduling=ahead)
        assert llm._ahead == ahead
        prompts, params = [], []
        for i in range(18):
            prompts.append(H.random_tokens(rng, rng.choice([1, 3, 16, 17, 40, 90]), cfg["vocab_size"]))
            params.append(SamplingParams(temperature=[0.0, 0.9, 0.7][i % 3], top_k=[-1, -1, 40][i % 3],
                                         max_tokens=rng.choice([1, 2, 7, 60, 100]), seed=500 + i,
                                         stop_token_ids=stops if i % 2 else [], ignore_eos=True))
        outs = llm.generate(prompts, params)
        llm.runner.check_device_status()
        llm.runner.manager.check_invariants()
        assert llm.runner.manager.num_free_blocks() == 13 and not llm.has_unfinished()
        assert llm.stats.generated_tokens == sum(len(o.output_ids) for o in outs)     # steps run in vain do not count
        for o, sp in zip(outs, params):
            assert 1 <= len(o.output_ids) <= sp.max_tokens
            assert all(0 <= t < cfg["vocab_size"] for t in o.output_ids)
            if o.finish_reason == "stop":
                assert o.output_ids[-1] in stops and not any(t in stops for t in o.output_ids[:-1])
            else:
                assert len(o.output_ids) == sp.max_tokens
        # whichever way the steps were launched, the greedy requests get the plain implementation's tokens
        greedy = [(p, o) for p, o, sp in zip(prompts, outs, params) if sp.temperature == 0.0]
        exact = sum(H.check_greedy(oracle, p, o.output_ids) for p, o in greedy)
        assert exact >= 0.9 * sum(len(o.output_ids) for _, o in greedy)
        return [(o.output_ids, o.finish_reason) for o in outs], llm.stats

    one, stats_one = run(False)
    two, stats_two = run(True)
    assert stats_two.preemptions > 0 and any(r == "stop" for _, r in two)
    if dtype == "float32":
        assert one == two


def test_logit_bias_and_logprobs_through_the_entry_point(dirs):
    """A bias of +100 on one token makes greedy generation emit it; log-probabilities come from the model's own
    logits (before the bias) and agree with the plain implementation: chosen token, rank, the most likely tokens."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_A
    W = H.load_plain_weights(dirs["A"])
    rng = random.Random(4)
    prompts = [H.random_tokens(rng, n, cfg["vocab_size"]) for n in (5, 9)]
    llm = LLM(dirs["A"], dtype="float32", max_model_len=64, max_num_seqs=4, max_num_batched_tokens=16,
              num_blocks=40, block_size=4)
    sp = [SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, logprobs=3),
          SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, logit_bias={17: 100.0}, logprobs=0)]
    outs = llm.generate(prompts, sp)
    assert outs[1].output_ids == [17] * 6
    for o, p, k in zip(outs, prompts, (3, 0)):
        assert len(o.logprobs) == 6
        seq = list(p)
        for t, rec in zip(o.output_ids, o.logprobs):
            lg = P.qwen3_logits(W, cfg, seq)[-1].double()
            want = torch.log_softmax(lg, dim=-1)
            assert rec.token_id == t and abs(rec.logprob - float(want[t])) < 1e-4
            assert rec.rank == int((lg > lg[t]).sum())
            assert len(rec.top_ids) == k
            if k:
                assert rec.top_ids == torch.topk(lg, k).indices.tolist()
                assert all(abs(a - float(want[i])) < 1e-4 for a, i in zip(rec.top_logprobs, rec.top_ids))
            seq.append(t)
    greedy = llm.generate(prompts[:1], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    assert greedy[0].logprobs is None and greedy[0].output_ids == outs[0].output_ids
    with pytest.raises(ValueError):
        llm.add_request([1, 2], SamplingParams(logit_bias={cfg["vocab_size"]: 1.0}))
    with pytest.raises(ValueError):
        llm.add_request([1, 2], SamplingParams(logprobs=33))


@pytest.mark.parametrize("seed", [2, 3, 10])
def test_scheduling_ahead_with_arrivals_and_aborts(dirs, seed):
    """Requests that arrive while others run, one aborted now and then (also with a step in flight), pools small
    enough to preempt: driven through ``step()`` one step at a time and one step ahead, 32-bit: the requests that
    were not aborted get the same tokens, and every page comes back."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_B
    rng0 = random.Random(seed)
    nb, seqs, budget = rng0.choice([12, 16]), rng0.choice([2, 4, 8]), rng0.choice([8, 32, 64])
    res = {}
    for ahead in (False, True):
        rng = random.Random(1000 + seed)
        llm = LLM(dirs["B"], dtype="float32", max_model_len=160, max_num_seqs=seqs, max_num_batched_tokens=budget,
                  num_blocks=nb, block_size=16, async_scheduling=ahead)
        stops = list(range(0, cfg["vocab_size"], rng.choice([15, 40, 200])))
        pending = []
        for i in range(rng.randint(12, 25)):
            mx = rng.choice([1, 2, 3, 10, 40])
            pending.append((H.random_tokens(rng, rng.choice([1, 2, 3, 15, 16, 17, 33, 64, 100]), cfg["vocab_size"]),
                            SamplingParams(temperature=rng.choice([0.0, 0.8, 1.0]), top_k=rng.choice([-1, 5, 40]),
                                           top_p=rng.choice([1.0, 0.9]), max_tokens=mx, min_tokens=min(mx, rng.choice([0, 0, 2])),
                                           seed=7 * i + seed, stop_token_ids=stops if rng.random() < 0.6 else [],
                                           ignore_eos=True)))
        ids, outs, aborted, step = [], {}, set(), 0
        while pending or llm.has_unfinished():
            for _ in range(rng.randint(0, 3)):
                if pending:
                    ids.append(llm.add_request(*pending.pop(0)))
            if step % 17 == 16 and ids:
                victim = ids[(step // 17) % len(ids)]
                if victim not in outs:
                    llm.abort(victim)
                    aborted.add(victim)
            for o in llm.step():
                outs[o.req_id] = o
            step += 1
            assert step < 5000
        llm.runner.manager.check_invariants()
        assert llm.runner.manager.num_free_blocks() == nb
        llm.runner.check_device_status()
        res[ahead] = ({i: (outs[i].output_ids, outs[i].finish_reason) for i in ids if i not in aborted}, aborted)
    # who gets aborted depends on the number of calls, which differs between the two ways: compare the others
    common = [i for i in res[False][0] if i in res[True][0]]
    assert common and all(res[False][0][i] == res[True][0][i] for i in common)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_budget_filling_steps_replay_a_graph(dirs, tmp_path, dtype):
    """Steps whose prompt portions fill the token budget exactly, and steps with few prompt tokens (padded up to a
    power of two by a dummy portion), replay a captured graph (one per number of prompt tokens and bucket of decoded
    tokens beside them, with places for up to four portions).  Against the same engine launching every such step
    kernel by kernel: the same tokens in 32-bit; in bfloat16 the same up to a near-tie."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_B if dtype == "float32" else H.TINY_D
    d = dirs["B"] if dtype == "float32" else H.make_model_dir(str(tmp_path / "d"), cfg, *H.INIT["D"], torch.bfloat16)
    rng = random.Random(21)
    # long prompts beside short ones: portions of one prompt, and the end of one with the start of the next
    prompts = [H.random_tokens(rng, n, cfg["vocab_size"]) for n in (100, 7, 90, 33, 64, 120, 5, 48, 80, 96)]
    sp = [SamplingParams(temperature=0.0 if i % 2 else 0.8, max_tokens=30, seed=40 + i, ignore_eos=True)
          for i in range(len(prompts))]
    res = {}
    for mixed in (False, True):
        llm = LLM(d, dtype=dtype, max_model_len=256, max_num_seqs=6, max_num_batched_tokens=32,
                  num_blocks=120, block_size=16, mixed_cuda_graph=mixed)
        res[mixed] = [o.output_ids for o in llm.generate(prompts, sp)]
        for n in (5, 7, 11, 20):                      # short prompts one after the other: 16, 16, 16, 32 prompt rows
            res[mixed] += [o.output_ids for o in llm.generate([prompts[0][:n]], sp[1])]
        captured = [k for k in llm.runner._graphs if isinstance(k, tuple)]
        assert bool(captured) == mixed
        if mixed:        # steps that fill the budget, and steps with few prompt tokens padded up to a power of two
            assert any(k[1] == 32 for k in captured) and any(k[1] < 32 for k in captured)
            assert llm.runner._padded_tokens >= 2048         # a tiny model: the host is always the slower side
        llm.runner.check_device_status()
        llm.runner.manager.check_invariants()
        assert llm.runner.manager.num_free_blocks() == 120
    if dtype == "float32":
        assert res[False] == res[True]
    else:
        agree = sum(a == b for x, y in zip(res[False], res[True]) for a, b in zip(x, y))
        assert agree >= 0.8 * sum(len(x) for x in res[False])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_whole_and_in_portions(tmp_path, dtype):
    """4,400 tokens through the step function whole, in portions of 512 (which replay the graph of budget-filling
    steps from the second one on) and in portions of 1000 launched kernel by kernel, then 40 tokens decoded one by
    one after each: page tables longer than the kernels' shared-memory slices, long histories behind a portion.
    The logits at the compared places (the last token of every third portion, every decoded token) against the
    plain implementation run over the whole sequence."""
    from dinfer_b200.config.engine_config import EngineConfig
    from dinfer_b200.engine.batch import StepEntry
    from dinfer_b200.engine.runner import ModelRunner
    cfg = dict(H.TINY_D, max_position_embeddings=8192, num_hidden_layers=2)
    d = H.make_model_dir(str(tmp_path / "long"), cfg, *H.INIT["D"], torch.float32 if dtype == "float32" else torch.bfloat16)
    rng = random.Random(8)
    toks = H.random_tokens(rng, 4440, cfg["vocab_size"])
    want = H.PlainOracle(d).logits(toks)
    n0 = 4400
    tol = H.TOLERANCE[dtype]
    for budget in (4608, 512, 1000):
        r = ModelRunner.from_dir(d, EngineConfig(max_model_len=4608, max_num_seqs=4, max_num_batched_tokens=budget,
                                                 num_blocks=4608 // 16 + 8, block_size=16, dtype=dtype))
        got, places = [], []
        at = 0
        while at < n0:
            n = min(budget, n0 - at)
            asked = at + n == n0 or (at // budget) % 3 == 0
            out = r.step([StepEntry("a", toks[at:at + n], [n - 1] if asked else [])])
            if asked:
                got.append(out[-1].float().cpu())
                places.append(at + n - 1)
            at += n
        for i, t in enumerate(toks[n0:]):
            got.append(r.step([StepEntry("a", [t], [0])])[0].float().cpu())
            places.append(n0 + i)
        if budget == 512:
            assert ("mixed", 512, 4, 0, False) in r._graphs          # the graph of portions beyond the short contexts
        r.finish("a")
        r.check_device_status()
        err = H.rel_err(torch.stack(got).numpy(), want[places])
        print("long prompt", dtype, budget, err)
        assert err <= tol, (budget, err)


def test_scheduling_ahead_with_the_prefix_cache_on(dirs):
    """Both of the reference's defaults together: one step in flight and the prefix cache.  Tokens a step took on
    the device reach the cache manager when the host reads them, so pages of generated tokens become findable
    too.  32-bit: the same tokens as one step at a time, prefix hits in both, every page back."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_B
    rng = random.Random(31)
    stem = H.random_tokens(rng, 50, cfg["vocab_size"])
    prompts = [stem[:rng.choice([20, 35, 50])] + H.random_tokens(rng, rng.choice([1, 5, 30]), cfg["vocab_size"])
               for _ in range(14)]
    sp = [SamplingParams(temperature=[0.0, 0.9][i % 2], max_tokens=rng.choice([3, 20, 45]), seed=90 + i,
                         ignore_eos=True) for i in range(len(prompts))]
    res = {}
    for ahead in (False, True):
        llm = LLM(dirs["B"], dtype="float32", max_model_len=160, max_num_seqs=4, max_num_batched_tokens=32,
                  num_blocks=24, block_size=16, enable_prefix_caching=True, async_scheduling=ahead)
        assert llm._ahead == ahead
        outs = llm.generate(prompts, sp)
        # a second round repeats the first request with what it generated: found in the cache
        rep = llm.generate([prompts[0] + outs[0].output_ids + [7]], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
        res[ahead] = ([o.output_ids for o in outs], rep[0].output_ids)
        assert llm.stats.prefix_hit_tokens > 0
        llm.runner.manager.check_invariants()
        assert llm.runner.manager.num_free_blocks() == 24
        llm.runner.check_device_status()
    assert res[False] == res[True]


def test_tokens_can_be_taken_step_by_step(dirs):
    """A caller that streams: after every ``step()`` the tokens each request got since the last look; put together
    they are the requests' outputs, with and without a step in flight."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_A
    rng = random.Random(2)
    prompts = [H.random_tokens(rng, n, cfg["vocab_size"]) for n in (3, 9, 14)]
    for ahead in (False, True):
        llm = LLM(dirs["A"], dtype="float32", max_model_len=64, max_num_seqs=4, max_num_batched_tokens=8,
                  num_blocks=40, block_size=4, async_scheduling=ahead)
        ids = [llm.add_request(p, SamplingParams(temperature=0.0, max_tokens=5 + i, stop_token_ids=[3, 7, 11]))
               for i, p in enumerate(prompts)]
        streamed = {i: [] for i in ids}
        done = {}
        while llm.has_unfinished():
            for o in llm.step():
                done[o.req_id] = o
            for rid, toks in llm.take_new_tokens().items():
                assert rid not in done or streamed[rid] + toks == done[rid].output_ids
                streamed[rid] += toks
        assert all(streamed[i] == done[i].output_ids for i in ids)
        assert llm.take_new_tokens() == {}


def test_prompt_logprobs(dirs):
    """Every prompt token but the first comes with its log-probability given the tokens before it, also when the
    prompt runs in portions beside other requests; against log_softmax of the plain implementation's logits."""
    from dinfer_b200 import LLM, SamplingParams
    cfg = H.TINY_A
    W = H.load_plain_weights(dirs["A"])
    rng = random.Random(6)
    prompts = [H.random_tokens(rng, n, cfg["vocab_size"]) for n in (11, 2, 1, 7)]
    llm = LLM(dirs["A"], dtype="float32", max_model_len=64, max_num_seqs=4, max_num_batched_tokens=4,
              num_blocks=40, block_size=4, enable_prefix_caching=True)
    sp = [SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True, prompt_logprobs=2),
          SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True, prompt_logprobs=0),
          SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True, prompt_logprobs=1),
          SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)]
    outs = llm.generate(prompts, sp)
    assert outs[3].prompt_logprobs is None
    for o, p, k in zip(outs[:3], prompts[:3], (2, 0, 1)):
        assert o.output_ids == P.greedy_generate(W, cfg, p, 3)
        assert len(o.prompt_logprobs) == len(p) and o.prompt_logprobs[0] is None
        if len(p) > 1:
            want = torch.log_softmax(P.qwen3_logits(W, cfg, p).double(), dim=-1)
            for i in range(1, len(p)):
                rec = o.prompt_logprobs[i]
                assert rec.token_id == p[i] and abs(rec.logprob - float(want[i - 1, p[i]])) < 1e-4
                assert rec.rank == int((want[i - 1] > want[i - 1, p[i]]).sum())
                assert rec.top_ids == torch.topk(want[i - 1], k).indices.tolist() if k else rec.top_ids == []
    llm.runner.manager.check_invariants()


def test_decode_graphs_in_the_measured_form(tmp_path):
    """split_norms = "auto": every decode bucket's graph is captured with the norms whole and taken apart, both are
    timed, one is kept; whichever it is, the decoded tokens' logits are the plain model's."""
    from dinfer_b200.config.engine_config import EngineConfig
    from dinfer_b200.engine.batch import StepEntry
    from dinfer_b200.engine.runner import ModelRunner
    cfg = H.TINY_D
    rng = random.Random(12)
    toks = {r: H.random_tokens(rng, n, cfg["vocab_size"]) for r, n in {"a": 30, "b": 21, "c": 26}.items()}
    d = H.make_model_dir(str(tmp_path / "d"), cfg, *H.INIT["D"], torch.bfloat16)
    oracle = H.PlainOracle(d)
    r = ModelRunner.from_dir(d, EngineConfig(max_model_len=64, max_num_seqs=4, max_num_batched_tokens=64,
                                                     num_blocks=16, block_size=16, dtype="bfloat16", split_norms="auto"))
    assert r.model.can_split_norms(4)
    buckets = [k for k in r._graphs if isinstance(k, int)]
    assert buckets == [1, 2, 4]                                      # captured when the engine starts
    for k in buckets:
        t_whole, t_apart = r._graphs[k]["times_ms"]
        assert t_whole > 0 and t_apart > 0
        assert r._graphs[k]["split_norms"] == (t_apart <= 0.98 * t_whole)
    assert r.split_norms_buckets() == [k for k in buckets if r._graphs[k]["split_norms"]]
    got = {k: [] for k in toks}
    out = r.step([StepEntry(k, t[:6], [5]) for k, t in toks.items()])
    for i, k in enumerate(toks):
        got[k].append(out[i].float().cpu())
    p = 6
    while any(len(t) > p for t in toks.values()):
        live = [k for k, t in toks.items() if len(t) > p]
        out = r.step([StepEntry(k, [toks[k][p]], [0]) for k in live])
        for j, k in enumerate(live):
            got[k].append(out[j].float().cpu())
            if len(toks[k]) == p + 1:
                r.finish(k)
        p += 1
    r.check_device_status()
    for k, t in toks.items():
        err = H.rel_err(torch.stack(got[k]).numpy(), oracle.logits(t)[5:])
        assert err <= H.TOLERANCE["bfloat16"], (k, err)
