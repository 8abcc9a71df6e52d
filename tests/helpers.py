"""Shared pieces of the tests: tiny configurations, model folders in a temporary place, the plain
oracle's logits, a driver of ``bin/trace_run`` and the ways a set of requests is cut into steps."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(__file__))

import plain_model  # noqa: E402

# Two (and a third) tiny configurations that differ in every size and option.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64,
              intermediate_size=160, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
              head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=128,
              tie_word_embeddings=True, attention_bias=False, hidden_act="silu", eos_token_id=7)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=517, hidden_size=96,
              intermediate_size=224, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2,
              head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0, max_position_embeddings=256,
              tie_word_embeddings=False, eos_token_id=[3, 5])
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=331, hidden_size=120,
              intermediate_size=200, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5,
              head_dim=48, rms_norm_eps=3e-6, rope_theta=50000.0, max_position_embeddings=512,
              tie_word_embeddings=False)
# Head geometries of the tensor-core kernels at a small width: head size 128 in groups of 4, head size 64 in
# groups of 2 (tcgen05 prompt attention, TMA decode attention, tcgen05 decode products, lane kernel of q/k).
TINY_D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1000, hidden_size=256,
              intermediate_size=384, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
              head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=1024,
              tie_word_embeddings=False)
TINY_E = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=777, hidden_size=192,
              intermediate_size=320, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
              head_dim=64, rms_norm_eps=2e-6, rope_theta=10000.0, max_position_embeddings=1024,
              tie_word_embeddings=True)
# init rules of the tiny models: (seed, std, norm jitter)
INIT = {"A": (0, 0.05, 0.1), "B": (1, 0.03, 0.2), "C": (2, 0.04, 0.15), "D": (3, 0.03, 0.1), "E": (4, 0.04, 0.1)}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def make_model_dir(path: str, cfg: dict, seed: int, std: float, jitter: float,
                   dtype: torch.dtype = torch.bfloat16, device: str = "cpu") -> str:
    from dinfer_b200.weights.random_init import write_random_model
    return write_random_model(path, cfg, seed, std, jitter, dtype, device=device)


def load_plain_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    """Read with the ``safetensors`` package, not with the engine's reader."""
    from safetensors.torch import load_file
    return load_file(os.path.join(model_dir, "model.safetensors"))


def random_tokens(rng: random.Random, n: int, vocab: int) -> List[int]:
    return [rng.randrange(vocab) for _ in range(n)]


class PlainOracle:
    """Logits of whole sequences by the plain implementation (64-bit), cached per sequence."""

    def __init__(self, model_dir: str):
        self.cfg = json.load(open(os.path.join(model_dir, "config.json")))
        self.W = load_plain_weights(model_dir)
        self._cache: Dict[Tuple[int, ...], np.ndarray] = {}

    def logits(self, ids: Sequence[int]) -> np.ndarray:
        key = tuple(ids)
        if key not in self._cache:
            self._cache[key] = plain_model.qwen3_logits(self.W, self.cfg, list(ids)).numpy()
        return self._cache[key]


def check_greedy(oracle: "PlainOracle", prompt: Sequence[int], output_ids: Sequence[int], rel: float = 0.05) -> int:
    """Every token of a greedy generation against the plain implementation run over the very sequence the engine
    produced: the token is the plain logits' largest entry, or (reduced precision may leave the path at a
    near-tie) lies within ``rel`` of the largest magnitude below it.  Returns how many were the largest."""
    seq = list(prompt) + list(output_ids)
    lg = oracle.logits(seq)
    exact = 0
    for i, t in enumerate(output_ids):
        row = lg[len(prompt) - 1 + i]
        top = int(row.argmax())
        if t == top:
            exact += 1
            continue
        gap = float(row[top] - row[t])
        assert gap < rel * float(np.abs(row).max()), (f"token {i} of the output is {t}, the plain implementation "
                                                      f"has {top}, {gap:.4f} above it (no near-tie)")
    return exact


class Replay:
    """One ``bin/trace_run`` process; ``step`` sends a line, waits for ``done`` and reads the file."""

    def __init__(self, model_dir: str, dtype: str, out_dir: str, max_tokens: int, extra: Sequence[str] = ()):
        self.out_dir = out_dir
        os.makedirs(out_dir, exist_ok=True)
        self.vocab = json.load(open(os.path.join(model_dir, "config.json")))["vocab_size"]
        self.proc = subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
             "--out", out_dir, "--max-tokens", str(max_tokens), *extra],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.n = 0

    def step(self, entries: List[dict], end: Sequence[str] = ()) -> Optional[np.ndarray]:
        step = self.n
        self.n += 1
        self.proc.stdin.write(json.dumps({"step": step, "entries": entries, "end": list(end)}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {step}":
            raise RuntimeError(f"trace_run answered {line!r} to step {step} (exit {self.proc.poll()})")
        wanted = sum(len(e.get("want", [])) for e in entries)
        if not wanted:
            return None
        a = np.fromfile(os.path.join(self.out_dir, f"{step}.f32"), dtype="<f4")
        return a.reshape(wanted, self.vocab)

    def close(self) -> int:
        self.proc.stdin.close()
        return self.proc.wait(timeout=120)


# ---------------------------------------------------------------- cutting requests into steps
# A schedule is a list of steps; a step is (entries, end) with entries = [(req, lo, hi)] meaning the
# tokens [lo, hi) of request ``req``.  Every position's logits are asked for.

def schedule_whole(lengths: Dict[str, int]):
    return [([(r, 0, n)], [r]) for r, n in lengths.items()]


def schedule_tail(lengths: Dict[str, int], tail: int = 32):
    steps = []
    for r, n in lengths.items():
        head = max(1, n - tail)
        steps.append(([(r, 0, head)], [r] if head == n else []))
        for p in range(head, n):
            steps.append(([(r, p, p + 1)], [r] if p == n - 1 else []))
    return steps


def schedule_chunks(lengths: Dict[str, int], rng: random.Random, sizes=(2, 3, 5, 8, 13, 2, 17, 4)):
    steps = []
    for r, n in lengths.items():
        p, i = 0, rng.randrange(len(sizes))
        while p < n:
            c = min(sizes[i % len(sizes)], n - p)
            i += 1
            steps.append(([(r, p, p + c)], [r] if p + c == n else []))
            p += c
    return steps


def schedule_mixed(lengths: Dict[str, int], rng: random.Random, max_live: int = 4, decode_tail: int = 12):
    """Up to ``max_live`` requests at a time: prompts in portions of 2..11 tokens beside single
    decoded tokens of others; a request may sit a step out; a finished one is replaced at once."""
    waiting = list(lengths)
    live: Dict[str, int] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for r in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                      # left out of this step, goes on later
            p, n = live[r], lengths[r]
            c = 1 if n - p <= decode_tail else min(rng.randrange(2, 12), n - p - decode_tail)
            entries.append((r, p, p + c))
            live[r] = p + c
            if p + c == n:
                end.append(r)
                del live[r]
        if entries:
            steps.append((entries, end))
    return steps


def schedule_mixed_large(lengths: Dict[str, int], rng: random.Random, portions=(40, 130, 512, 700),
                         max_live: int = 4, decode_tail: int = 14, admit_every: int = 3):
    """The steps a serving engine runs: up to ``max_live`` requests, prompts in LARGE portions (drawn from
    ``portions``, so that a step's rows reach every product path: up to 32, 33..511, 512 and more) beside single
    decoded tokens of the others; the last ``decode_tail`` tokens of every request come one by one.  A new request
    is let in every ``admit_every`` steps at the earliest, so that its portions meet the others' decoded tokens;
    a request may sit a step out; a finished one makes room, so pages are used again."""
    waiting = list(lengths)
    live: Dict[str, int] = {}
    steps = []
    since = admit_every
    while waiting or live:
        if waiting and len(live) < max_live and (since >= admit_every or not live):
            live[waiting.pop(0)] = 0
            since = 0
        since += 1
        entries, end = [], []
        for r in list(live):
            p, n = live[r], lengths[r]
            left = n - p - decode_tail
            if left <= 1 and len(live) > 1 and rng.random() < 0.15:
                continue                                   # a decoding request sits this step out
            c = 1 if left <= 1 else min(rng.choice(portions), left)
            entries.append((r, p, p + c))
            live[r] = p + c
            if p + c == n:
                end.append(r)
                del live[r]
        if entries:
            steps.append((entries, end))
    return steps


def schedule_rolling(names: Sequence[str], portions: Sequence[int], n_decode: int, stagger: int = 1):
    """Requests that are all alike, one starting every ``stagger`` steps: the prompt in ``portions`` (one a step),
    then ``n_decode`` tokens one a step.  In the steady state every step has the same shape (the same portions
    beside the same number of decoded tokens), which is what a captured graph of such a step needs to be replayed.
    Returns (steps, lengths)."""
    plan = list(portions) + [1] * n_decode
    n_steps = (len(names) - 1) * stagger + len(plan)
    steps = []
    for t in range(n_steps):
        entries, end = [], []
        for i, r in enumerate(names):
            k = t - i * stagger
            if 0 <= k < len(plan):
                lo = sum(plan[:k])
                entries.append((r, lo, lo + plan[k]))
                if k == len(plan) - 1:
                    end.append(r)
        steps.append((entries, end))
    return steps, {r: sum(plan) for r in names}


def max_live_tokens(steps, round_to: int = 64) -> int:
    """Most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: Dict[str, int] = {}
    worst = 0
    for entries, end in steps:
        for r, lo, hi in entries:
            held[r] = hi
        worst = max(worst, sum((v + round_to - 1) // round_to * round_to for v in held.values()))
        for r in end:
            held.pop(r, None)
    return worst


def run_schedule(replay: Replay, steps, tokens: Dict[str, List[int]], tag: str = ""):
    """Replays the steps; returns {req: [n, V] logits} assembled from the steps' outputs."""
    got = {r: np.full((len(t), replay.vocab), np.nan, dtype=np.float32) for r, t in tokens.items()}
    for entries, end in steps:
        ents = [{"id": tag + r, "tokens": tokens[r][lo:hi], "want": list(range(hi - lo))} for r, lo, hi in entries]
        out = replay.step(ents, [tag + r for r in end])
        o = 0
        for r, lo, hi in entries:
            got[r][lo:hi] = out[o:o + hi - lo]
            o += hi - lo
    return got


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """Largest difference over the largest magnitude of the expected logits."""
    if not np.isfinite(got).all():
        return float("inf")
    return float(np.abs(got.astype(np.float64) - want).max() / np.abs(want).max())


# one tolerance per dtype, fixed before the first run
TOLERANCE = {"float32": 1e-4, "bfloat16": 2e-2}


class LocalReplay:
    """The same ``step`` interface as ``Replay`` on a ModelRunner of this process (for architectures
    that exist only in the test that registers them)."""

    def __init__(self, model_dir: str, dtype: str, max_tokens: int, block_size: int = 16, **engine):
        from dinfer_b200.config.engine_config import EngineConfig
        from dinfer_b200.engine.runner import ModelRunner
        cfg = json.load(open(os.path.join(model_dir, "config.json")))
        self.vocab = cfg["vocab_size"]
        n = (max_tokens + 63) // 64 * 64
        self.runner = ModelRunner.from_dir(model_dir, EngineConfig(
            max_model_len=min(n, cfg.get("max_position_embeddings", cfg.get("max_positions", n))), max_num_seqs=16,
            max_num_batched_tokens=n, num_blocks=n // block_size, block_size=block_size, dtype=dtype,
            enable_cuda_graph=False, **engine))

    def step(self, entries: List[dict], end: Sequence[str] = ()) -> Optional[np.ndarray]:
        from dinfer_b200.engine.batch import StepEntry
        out = self.runner.step([StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in entries])
        for r in end:
            self.runner.finish(r)
        return out.cpu().numpy() if out.shape[0] else None

    def close(self) -> int:
        self.runner.manager.check_invariants()
        assert not self.runner.manager.requests()
        return 0
