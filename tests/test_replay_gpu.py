"""Trace replay against the plain implementation: each request whole; most of it in one step and
the last 32 tokens one by one; in portions of changing size down to two tokens; and mixed, up to
four live requests with so few pages that they are used again.  In 32-bit and in bfloat16, on
tiny configurations that differ in every size."""
import random

import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

LENGTHS = {
    "A": {"a": 1, "b": 7, "c": 19, "d": 64, "e": 97, "f": 128},
    "B": {"a": 3, "b": 16, "c": 17, "d": 40, "e": 63, "f": 150, "g": 255},
    "C": {"a": 2, "b": 33, "c": 129, "d": 200},
    "D": {"a": 5, "b": 100, "c": 300, "d": 515},          # several 64-key tiles per request
    "E": {"a": 3, "b": 64, "c": 257, "d": 450},
}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    out = {}
    for name, cfg in H.CONFIGS.items():
        seed, std, jit = H.INIT[name]
        for dt, tdt in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            d = tmp_path_factory.mktemp(f"tiny{name}_{dt}")
            out[(name, dt)] = H.make_model_dir(str(d), cfg, seed, std, jit, tdt)
    return out


@pytest.mark.parametrize("block_size", [4, 16, 32])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_replay_all_ways(model_dirs, tmp_path, name, dtype, block_size):
    """Pages of 4 tokens are Tiny A's own setting and put the decode attention for small pages (which folds its
    key splits through scratch memory) inside a whole model at head sizes 64 and 128; 16 is the default; 32 halves
    the pages of a 64-key tile."""
    model_dir = model_dirs[(name, dtype)]
    cfg = H.CONFIGS[name]
    rng = random.Random(1234 + ord(name))
    tokens = {r: H.random_tokens(rng, n, cfg["vocab_size"]) for r, n in LENGTHS[name].items()}
    oracle = H.PlainOracle(model_dir)
    want = {r: oracle.logits(t) for r, t in tokens.items()}
    lengths = LENGTHS[name]
    schedules = {
        "whole": H.schedule_whole(lengths),
        "tail32": H.schedule_tail(lengths, 32),
        "chunks": H.schedule_chunks(lengths, rng),
        "mixed": H.schedule_mixed(lengths, rng),
        "mixed2": H.schedule_mixed(dict(reversed(list(lengths.items()))), rng, max_live=3, decode_tail=33),
    }
    # the pool holds just what the most demanding schedule needs, so pages are used again
    max_tokens = max(H.max_live_tokens(s) for s in schedules.values())
    rp = H.Replay(model_dir, dtype, str(tmp_path / "out"), max_tokens, extra=["--block-size", str(block_size)])
    worst = {}
    try:
        for sname, steps in schedules.items():
            got = H.run_schedule(rp, steps, tokens, tag=sname + "/")
            worst[sname] = max(H.rel_err(got[r], want[r]) for r in tokens)
    finally:
        assert rp.close() == 0
    print(name, dtype, block_size, worst)
    tol = H.TOLERANCE[dtype]
    bad = {k: v for k, v in worst.items() if not v <= tol}
    assert not bad, f"{name} {dtype} pages of {block_size}: relative error above {tol}: {bad} (all: {worst})"


LARGE = {"D": {"a": 1000, "b": 640, "c": 777, "d": 1024, "e": 600, "f": 913},
         "E": {"a": 655, "b": 1024, "c": 600, "d": 870, "e": 731}}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_replay_large_portions_beside_decoded_tokens(model_dirs, tmp_path, name, dtype):
    """What a serving engine runs: prompts of 600 to 1024 tokens taken in portions of 40, 130, 512 and 700 tokens
    BESIDE single decoded tokens of up to three other requests, so that a step's rows reach every product path
    (up to 32 rows, 33 to 511, 512 and more) and the prompt and the decode attention kernels run on one batch;
    the pool holds what the live requests need, so pages are used again.  Every position's logits against the
    plain implementation (the reference tests such batches at kernel level:
    crates/kernels/tests/ops_parity.rs:716-739, and through its engine: models/qwen3/tests/real_parity.rs:293-309)."""
    model_dir = model_dirs[(name, dtype)]
    cfg = H.CONFIGS[name]
    rng = random.Random(77 + ord(name))
    lengths = LARGE[name]
    tokens = {r: H.random_tokens(rng, n, cfg["vocab_size"]) for r, n in lengths.items()}
    oracle = H.PlainOracle(model_dir)
    want = {r: oracle.logits(t) for r, t in tokens.items()}
    schedules = {"large": H.schedule_mixed_large(lengths, rng),
                 "large3": H.schedule_mixed_large(dict(reversed(list(lengths.items()))), rng, portions=(512, 33, 700, 2),
                                                  max_live=3, decode_tail=25)}
    for steps in schedules.values():                # the steps are what the test is named for
        rows = [sum(hi - lo for _, lo, hi in e) for e, _ in steps if any(hi - lo == 1 for _, lo, hi in e)]
        assert any(r >= 512 for r in rows) and any(33 <= r < 512 for r in rows)
    rp = H.Replay(model_dir, dtype, str(tmp_path / "out"), max(H.max_live_tokens(s) for s in schedules.values()))
    worst = {}
    try:
        for sname, steps in schedules.items():
            got = H.run_schedule(rp, steps, tokens, tag=sname + "/")
            worst[sname] = max(H.rel_err(got[r], want[r]) for r in tokens)
    finally:
        assert rp.close() == 0
    print(name, dtype, worst)
    assert all(v <= H.TOLERANCE[dtype] for v in worst.values()), worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_graph_replayed_steps_with_prompt_portions_against_the_plain_model(model_dirs, name, dtype):
    """Steps with prompt portions that replay a captured graph (laid out as prompt places, one of them a dummy
    portion that pads the step, and a bucket of one-token places), each shape many times: portions that fill the
    token budget exactly; few prompt tokens padded to a power of two; more, padded to a multiple of 128; more
    than four portions (the 16-place layout).  Decoded tokens of other requests ride in every step; the logits
    of every entry's last token against the plain implementation."""
    from dinfer_b200.config.engine_config import EngineConfig
    from dinfer_b200.engine.batch import StepEntry
    from dinfer_b200.engine.runner import ModelRunner
    model_dir = model_dirs[(name, dtype)]
    cfg = H.CONFIGS[name]
    rng = random.Random(5 + ord(name))
    oracle = H.PlainOracle(model_dir)
    workloads = [([256, 256, 256], 4), ([50, 40], 3), ([300, 200], 2), ([20] * 5, 1)]
    plans = [H.schedule_rolling([f"w{k}r{i}" for i in range(12)], portions, n_dec)
             for k, (portions, n_dec) in enumerate(workloads)]
    pool = max(H.max_live_tokens(steps) for steps, _ in plans)
    r = ModelRunner.from_dir(model_dir, EngineConfig(
        max_model_len=1024, max_num_seqs=8, max_num_batched_tokens=768, num_blocks=pool // 16, block_size=16,
        dtype=dtype, enable_cuda_graph=True, mixed_cuda_graph=True))
    replays = {}
    inner = r._mixed_graph_step

    def counted(entries, starts, key, places):
        replays[key] = replays.get(key, 0) + 1
        return inner(entries, starts, key, places)

    r._mixed_graph_step = counted
    worst = 0.0
    for steps, lengths in plans:
        tokens = {q: H.random_tokens(rng, n, cfg["vocab_size"]) for q, n in lengths.items()}
        for entries, end in steps:
            out = r.step([StepEntry(q, tokens[q][lo:hi], [hi - lo - 1]) for q, lo, hi in entries]).cpu().numpy()
            for i, (q, lo, hi) in enumerate(entries):
                worst = max(worst, H.rel_err(out[i], oracle.logits(tokens[q])[hi - 1]))
            for q in end:
                r.finish(q)
        r.check_device_status()
    r.manager.check_invariants()
    assert r.manager.num_free_blocks() == pool // 16
    shapes = {(k[1], k[2]) for k in replays}
    # budget filled exactly (768), padded to a power of two (128), to a multiple of 128 (512), 16 places
    assert {(768, 4), (128, 4), (512, 4), (128, 16)} <= shapes, replays
    for shape in ((768, 4), (128, 4), (512, 4), (128, 16)):          # each replayed many times with one bucket
        assert max(n for k, n in replays.items() if (k[1], k[2]) == shape) >= 3, replays
    print(name, dtype, worst, replays)
    assert worst <= H.TOLERANCE[dtype], worst


# The layer sizes of the benchmark shape (hidden 4096, 32 / 8 heads of 128, intermediate 12288), two layers and a
# shorter vocabulary so that the plain implementation stays affordable on the CPU.
LAYER_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=20011, hidden_size=4096,
                intermediate_size=12288, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960,
                tie_word_embeddings=False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_at_the_benchmark_layer_sizes(tmp_path, dtype):
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    model_dir = H.make_model_dir(str(tmp_path / "m8b"), LAYER_8B, 42, 0.02, 0.0, tdt)
    rng = random.Random(88)
    lengths = {"a": 70, "b": 33, "c": 2}
    tokens = {r: H.random_tokens(rng, n, LAYER_8B["vocab_size"]) for r, n in lengths.items()}
    oracle = H.PlainOracle(model_dir)
    want = {r: oracle.logits(t) for r, t in tokens.items()}
    schedules = {"whole": H.schedule_whole(lengths), "tail32": H.schedule_tail(lengths, 32),
                 "chunks": H.schedule_chunks(lengths, rng),
                 "mixed": H.schedule_mixed(lengths, rng, max_live=3, decode_tail=9)}
    rp = H.LocalReplay(model_dir, dtype, max(H.max_live_tokens(s) for s in schedules.values()))
    worst = {}
    try:
        for sname, steps in schedules.items():
            got = H.run_schedule(rp, steps, tokens, tag=sname + "/")
            worst[sname] = max(H.rel_err(got[r], want[r]) for r in tokens)
    finally:
        assert rp.close() == 0
    print("8B layer sizes", dtype, worst)
    assert all(v <= H.TOLERANCE[dtype] for v in worst.values()), worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_with_the_benchmark_vocabulary(tmp_path, dtype):
    """One layer of the benchmark shape with its real vocabulary of 151,936 (no power of two; the embedding and
    the head at their true sizes, untied): whole, in portions down to two tokens, and mixed."""
    cfg = dict(LAYER_8B, vocab_size=151936, num_hidden_layers=1)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    model_dir = H.make_model_dir(str(tmp_path / "mv"), cfg, 43, 0.02, 0.0, tdt, device="cuda")
    rng = random.Random(89)
    lengths = {"a": 41, "b": 18, "c": 2}
    tokens = {r: H.random_tokens(rng, n, cfg["vocab_size"]) for r, n in lengths.items()}
    tokens["a"][3], tokens["b"][0] = cfg["vocab_size"] - 1, 0             # the table's last and first rows
    oracle = H.PlainOracle(model_dir)
    want = {r: oracle.logits(t) for r, t in tokens.items()}
    del oracle
    schedules = {"whole": H.schedule_whole(lengths), "chunks": H.schedule_chunks(lengths, rng),
                 "mixed": H.schedule_mixed(lengths, rng, max_live=3, decode_tail=9)}
    rp = H.LocalReplay(model_dir, dtype, max(H.max_live_tokens(s) for s in schedules.values()))
    worst = {}
    try:
        for sname, steps in schedules.items():
            got = H.run_schedule(rp, steps, tokens, tag=sname + "/")
            worst[sname] = max(H.rel_err(got[r], want[r]) for r in tokens)
    finally:
        assert rp.close() == 0
    import shutil
    shutil.rmtree(model_dir, ignore_errors=True)             # gigabytes: not left for the next test's disk
    print("benchmark vocabulary", dtype, worst)
    assert all(v <= H.TOLERANCE[dtype] for v in worst.values()), worst


@pytest.mark.parametrize("name", ["D", "E"])
def test_replay_with_the_norms_taken_apart(model_dirs, name):
    """The steps of at most 32 tokens (decoded tokens, small portions, mixed) with every norm between two
    products taken apart into their epilogues (bfloat16; the engine otherwise chooses by measurement)."""
    model_dir = model_dirs[(name, "bfloat16")]
    cfg = H.CONFIGS[name]
    rng = random.Random(4321 + ord(name))
    lengths = {"a": 5, "b": 100, "c": 290}
    tokens = {r: H.random_tokens(rng, n, cfg["vocab_size"]) for r, n in lengths.items()}
    oracle = H.PlainOracle(model_dir)
    want = {r: oracle.logits(t) for r, t in tokens.items()}
    schedules = {"tail32": H.schedule_tail(lengths, 32), "chunks": H.schedule_chunks(lengths, rng),
                 "mixed": H.schedule_mixed(lengths, rng, max_live=3, decode_tail=20)}
    rp = H.LocalReplay(model_dir, "bfloat16", max(H.max_live_tokens(s) for s in schedules.values()), split_norms=True)
    assert rp.runner.model.can_split_norms(8)
    worst = {}
    try:
        for sname, steps in schedules.items():
            got = H.run_schedule(rp, steps, tokens, tag=sname + "/")
            worst[sname] = max(H.rel_err(got[r], want[r]) for r in tokens)
    finally:
        assert rp.close() == 0
    print(name, "split norms", worst)
    assert all(v <= H.TOLERANCE["bfloat16"] for v in worst.values()), worst
