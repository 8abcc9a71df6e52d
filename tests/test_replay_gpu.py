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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_replay_all_ways(model_dirs, tmp_path, name, dtype):
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
    rp = H.Replay(model_dir, dtype, str(tmp_path / "out"), max_tokens)
    worst = {}
    try:
        for sname, steps in schedules.items():
            got = H.run_schedule(rp, steps, tokens, tag=sname + "/")
            worst[sname] = max(H.rel_err(got[r], want[r]) for r in tokens)
    finally:
        assert rp.close() == 0
    print(name, dtype, worst)
    tol = H.TOLERANCE[dtype]
    bad = {k: v for k, v in worst.items() if not v <= tol}
    assert not bad, f"{name} {dtype}: relative error above {tol}: {bad} (all: {worst})"


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
