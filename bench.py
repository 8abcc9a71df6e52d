#!/usr/bin/env python3
"""Benchmark of the engine on one GPU: decode tokens/s of a Qwen3-8B-shaped model with random
weights (batch 8, context 4096 by default), prefill tokens/s of one 2048-token prompt, and the
fraction of the memory / tensor-core roofline each reaches.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch B] [--context C] [--layers L]
    python bench.py --shape 32b             # the same at the Qwen3-32B (or 0.6b) layer sizes
    python bench.py --serving               # 32 requests through LLM.generate at the Qwen3-0.6B shape
    python bench.py --shape 0.6b --closed-loop 8,128,128    # the reference's "c8 p128 o128" at engine level
    python bench.py --impl reference        # the reference engine, where it can be installed

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  ``value`` times K steps on
the device (CUDA events); ``e2e`` is the same K steps through the Python entry point ``LLM.step()``,
each step copying its plan (token ids, positions, page tables) host->device from pinned memory and
reading sampled tokens device->host; the engine keeps one step in flight (it launches a step, then
reads the tokens of the step before), so K calls cover K steps' launches, copies and read-backs.
The cache is filled by really prefilling the prompts through the engine.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen3-8B shape: the benchmark configuration
QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
                intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960,
                tie_word_embeddings=False, attention_bias=False, hidden_act="silu")
# the other two shapes the reference's architecture is quoted at (python bench.py --shape ...)
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64)
QWEN3_06B = dict(QWEN3_8B, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 tie_word_embeddings=True)
SHAPES = {"8b": ("Qwen3-8B shape", QWEN3_8B), "32b": ("Qwen3-32B shape", QWEN3_32B), "0.6b": ("Qwen3-0.6B shape", QWEN3_06B)}
FULL_LAYERS = 36
PREFILL_TOKENS = 2048


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def model_numbers(cfg, layers):
    h, I, H, Hkv, D, V = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"],
                          cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"])
    per_layer = (H + 2 * Hkv) * D * h + h * H * D + 3 * I * h            # linear parameters
    norms = 2 * h + 2 * D
    weight_bytes = 2 * (layers * (per_layer + norms) + V * h + h)         # read once per decode step (bf16)
    kv_bytes_per_token = layers * 2 * Hkv * D * 2
    return dict(per_layer=per_layer, weight_bytes=weight_bytes, kv_bytes_per_token=kv_bytes_per_token)


def prefill_flops(cfg, layers, T):
    n = model_numbers(cfg, layers)
    H, D, V, h = cfg["num_attention_heads"], cfg["head_dim"], cfg["vocab_size"], cfg["hidden_size"]
    return 2.0 * T * n["per_layer"] * layers + layers * 2.0 * T * T * H * D + 2.0 * V * h


def make_llm(cfg, layers, max_seqs, context, seed=42, **engine):
    from dinfer_b200 import LLM
    from dinfer_b200.weights.random_init import RandomSource
    c = dict(cfg, num_hidden_layers=layers)
    blocks = max_seqs * ((context + 64 + 15) // 16) + (PREFILL_TOKENS + 64) // 16 + 64
    return LLM(config=c, weights=RandomSource(c, seed, std=0.02, norm_jitter=0.0), dtype="bfloat16",
               max_model_len=max(context, PREFILL_TOKENS) + 64, max_num_seqs=max(max_seqs, 1), max_num_batched_tokens=2048,
               num_blocks=blocks, block_size=16, enable_cuda_graph=True, **{"split_norms": "auto", **engine})


def count_launches(fn):
    """Kernel launches of ``fn()``: every call into this package's kernel libraries and every library
    matrix product counts one (a replayed CUDA graph counts the launches it captured)."""
    from dinfer_b200.kernels import lib
    n0 = lib.launch_count()
    fn()
    return lib.launch_count() - n0


def decode_run(llm, cfg, batch, context, steps, warmup, rng, measure_e2e, want_launches=False):
    """Prefill ``batch`` prompts so that the timed steps end at ``context`` tokens, then time decode."""
    import torch
    from dinfer_b200 import SamplingParams
    V = cfg["vocab_size"]
    total_steps = warmup + (steps if measure_e2e else 1)
    # requests that finish their prompt early decode while the others still prefill (two portions each),
    # so leave room for that drift; the bytes of the roofline use the contexts actually reached
    prompt_len = context - total_steps - 2 * batch - 1
    sp = SamplingParams(temperature=0.0, max_tokens=1 << 20, ignore_eos=True)
    for _ in range(batch):
        llm.add_request([rng.randrange(V) for _ in range(prompt_len)], sp)
    while any(r.num_computed < len(r.prompt_ids) for r in llm._requests.values()) or llm.scheduler.waiting:
        llm.step()
    for _ in range(warmup):
        llm.step()
    res = {}
    torch.cuda.synchronize()
    sampler = ClockSampler()
    sampler.start()
    if measure_e2e:
        # end to end: K steps through the Python entry point; every step copies its plan (token ids,
        # positions, page tables) host->device from pinned memory and reads the sampled tokens back
        host0 = (llm.stats.host_schedule_s, llm.stats.host_launch_s, llm.stats.host_collect_s)
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        res["e2e_ms_per_step"] = (time.perf_counter() - t0) * 1e3 / steps
        st = llm.stats
        res["host_us"] = [round((x - y) * 1e6 / steps, 1) for x, y in zip(
            (st.host_schedule_s, st.host_launch_s, st.host_collect_s), host0)]
        res["h2d_bytes_per_step"] = llm.runner.plan.h2d_bytes
        res["d2h_bytes_per_step"] = 4 * batch
    else:
        llm.step()
    # device time of one decode step: the step's captured graph (forward of the whole batch) replayed K
    # times back to back at the context just reached, timed with CUDA events, no host in between
    res["mean_context"] = sum(r.num_tokens + r.num_placeholders for r in llm._requests.values()) / batch - 1
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    from dinfer_b200.kernels import lib as _lib
    l0 = _lib.launch_count()
    e0.record()
    from dinfer_b200.sampling.sampler import argmax
    tokens = torch.empty(llm.runner.engine.max_num_seqs, dtype=torch.int32, device=llm.runner.device)
    llm.runner.replay_last_decode(steps, after=lambda logits: argmax(logits[:batch], out=tokens[:batch]))
    e1.record()
    torch.cuda.synchronize()
    res["ms_per_step"] = e0.elapsed_time(e1) / steps
    res["launches_per_step"] = (_lib.launch_count() - l0) // steps
    res["clocks"] = sampler.stop()
    for rid in list(llm._requests):
        llm.abort(rid)
    return res


def prefill_run(llm, cfg, tokens, rng, reps=3):
    import torch
    from dinfer_b200.engine.batch import StepEntry
    V = cfg["vocab_size"]
    best = None
    for i in range(reps + 1):
        ids = [rng.randrange(V) for _ in range(tokens)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        llm.runner.step([StepEntry(("prefill", i), ids, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        llm.runner.finish(("prefill", i))
        ms = e0.elapsed_time(e1)
        if i > 0:
            best = ms if best is None else min(best, ms)
    return best


def profile_region(a) -> int:
    """For a profiler: set up a small case, then bracket ONE decode step (or one prefill step) with
    cudaProfilerStart/Stop, so that ``ncu --profile-from-start off`` sees only that step's kernels.
    Prints no benchmark line: a run under a profiler is never a measurement."""
    import torch
    from dinfer_b200 import SamplingParams
    from dinfer_b200.engine.batch import StepEntry
    cfg = QWEN3_8B
    rng = random.Random(42)
    # the bracketed prefill step launches its kernels one by one (a profiler then lists them once, in order)
    llm = make_llm(cfg, a.layers, max(a.batch, 1), a.context, mixed_cuda_graph=False)
    V = cfg["vocab_size"]
    if a.profile == "prefill":
        ids = [rng.randrange(V) for _ in range(PREFILL_TOKENS)]
        llm.runner.step([StepEntry("w", ids, [PREFILL_TOKENS - 1])])
        llm.runner.finish("w")
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        llm.runner.step([StepEntry("p", ids, [PREFILL_TOKENS - 1])])
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return 0
    sp = SamplingParams(temperature=0.0, max_tokens=1 << 20, ignore_eos=True)
    for _ in range(a.batch):
        llm.add_request([rng.randrange(V) for _ in range(a.context - 16)], sp)
    while any(r.num_computed < len(r.prompt_ids) for r in llm._requests.values()) or llm.scheduler.waiting:
        llm.step()
    for _ in range(3):
        llm.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    llm.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return 0


def serving_run() -> int:
    """32 requests with prompts of 16..1024 tokens (seed 3) through ``LLM.generate`` at the Qwen3-0.6B shape:
    prompts cut into portions of 512 tokens beside decoding requests, 256 tokens each at temperature 0.7."""
    import torch
    from dinfer_b200 import LLM, SamplingParams
    from dinfer_b200.weights.random_init import RandomSource
    cfg = QWEN3_06B
    llm = LLM(config=cfg, weights=RandomSource(cfg, 3, std=0.02, norm_jitter=0.0), dtype="bfloat16", max_model_len=2048,
              max_num_seqs=32, max_num_batched_tokens=512, num_blocks=32 * 129, block_size=16)
    rng = random.Random(3)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(16, 1024))] for _ in range(32)]
    sp = [SamplingParams(temperature=0.7, max_tokens=256, ignore_eos=True, seed=100 + i) for i in range(32)]
    best = None
    for _ in range(3):                                  # the first pass also captures the decode graphs
        steps0 = llm.stats.steps
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        gen = sum(len(o.output_ids) for o in outs)
        mid = len(outs) // 2
        rec = {"seconds": round(dt, 4), "steps": llm.stats.steps - steps0, "generated": gen,
               # as the reference's bench reports them: time to the first token and time per token after it, medians
               "ttft_ms_p50": round(sorted(o.ttft_s for o in outs)[mid] * 1e3, 2),
               "tpot_ms_p50": round(sorted(o.tpot_s for o in outs)[mid] * 1e3, 3)}
        if best is None or dt < best["seconds"]:
            best = rec
    print(json.dumps({"metric": "serving: generated tok/s (Qwen3-0.6B shape, bf16, 32 requests, prompts 16..1024, "
                                "portions of 512, 256 tokens each at temperature 0.7)",
                      "value": round(best["generated"] / best["seconds"], 1), "unit": "tokens/s",
                      "prompt_tokens": sum(map(len, prompts)), "ms_per_step": round(best["seconds"] * 1e3 / best["steps"], 3),
                      **best, "impl": "ours", "data": "synthetic"}))
    return 0


def closed_loop_run(shape: str, clients: int, prompt_len: int, output_len: int, requests_per_client: int = 6) -> int:
    """The reference's serving measurement without the HTTP in between (its ``bench`` tool,
    scripts/verify/bench_compare.sh: "cN pP oO" = N clients, each sending its next request when the last has ended,
    prompts of P tokens, O generated tokens, temperature 0, ignore_eos, the first 2 requests of each client left
    out): output tokens a second over the measured requests, time to the first token and time per token after it."""
    import torch
    from dinfer_b200 import LLM, SamplingParams
    from dinfer_b200.weights.random_init import RandomSource
    name, cfg = SHAPES[shape]
    llm = LLM(config=cfg, weights=RandomSource(cfg, 3, std=0.02, norm_jitter=0.0), dtype="bfloat16",
              max_model_len=max(2048, prompt_len + output_len + 64), max_num_seqs=max(16, clients),
              max_num_batched_tokens=2048, block_size=16, split_norms="auto")
    rng = random.Random(11)
    sp = SamplingParams(temperature=0.0, max_tokens=output_len, ignore_eos=True)

    def prompt():
        return [rng.randrange(cfg["vocab_size"]) for _ in range(prompt_len)]
    sent = {c: 0 for c in range(clients)}
    owner, outs = {}, []
    for c in range(clients):
        owner[llm.add_request(prompt(), sp)] = c
        sent[c] += 1
    t_start = None
    while llm.has_unfinished():
        for o in llm.step():
            c = owner.pop(o.req_id)
            if sent[c] > 2:                                   # measured (the first two of a client warm up)
                outs.append(o)
            if sent[c] == 2 and t_start is None and all(n >= 2 for n in sent.values()):
                torch.cuda.synchronize()
                t_start = time.perf_counter()
            if sent[c] < requests_per_client:
                owner[llm.add_request(prompt(), sp)] = c
                sent[c] += 1
    torch.cuda.synchronize()
    dt = time.perf_counter() - (t_start or 0.0)
    gen = sum(len(o.output_ids) for o in outs)
    mid = len(outs) // 2
    print(json.dumps({"metric": f"closed loop c{clients} p{prompt_len} o{output_len}: output tok/s ({name}, bf16, random "
                                "weights, engine level, no HTTP)",
                      "value": round(gen / dt, 1), "unit": "tokens/s", "requests": len(outs),
                      "ttft_ms_p50": round(sorted(o.ttft_s for o in outs)[mid] * 1e3, 2),
                      "tpot_ms_p50": round(sorted(o.tpot_s for o in outs)[mid] * 1e3, 3),
                      "e2e_ms_p50": round(sorted(o.e2e_s for o in outs)[mid] * 1e3, 1),
                      "seconds": round(dt, 3), "impl": "ours", "data": "synthetic"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile", choices=["decode", "prefill"], default=None,
                    help="run one bracketed step for a profiler instead of the benchmark")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS)
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="8b", help="layer sizes of the model (default: the benchmark's)")
    ap.add_argument("--serving", action="store_true",
                    help="the mixed serving workload instead: 32 requests, prompts of 16..1024 tokens, portions of "
                         "512, 256 tokens each at temperature 0.7, at the Qwen3-0.6B shape")
    ap.add_argument("--closed-loop", default=None, metavar="C,P,O",
                    help="the reference's serving measurement at engine level instead: C clients, each sending its "
                         "next request when the last has ended, prompts of P tokens, O generated tokens (--shape applies)")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "rayze-ai/dinfer is a Rust workspace: no cargo/rustc in this image and pip finds no "
                          "Python project in it (no setup.py / pyproject.toml), so it cannot be installed offline"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    import torch
    if a.profile:
        return profile_region(a)
    if a.serving:
        return serving_run()
    if a.closed_loop:
        c, p_len, o_len = (int(x) for x in a.closed_loop.split(","))
        return closed_loop_run(a.shape, c, p_len, o_len)
    shape_name, cfg = SHAPES[a.shape]
    full_layers = cfg["num_hidden_layers"]
    if a.shape != "8b" and a.layers == FULL_LAYERS:
        a.layers = full_layers
    pk = peaks()
    rng = random.Random(42)
    nums = model_numbers(cfg, a.layers)
    llm = make_llm(cfg, a.layers, max(a.batch, 1 if a.no_points else 64), a.context)

    main_run = decode_run(llm, cfg, a.batch, a.context, a.steps, a.warmup, rng, measure_e2e=True, want_launches=True)
    ms = main_run["ms_per_step"]
    value = a.batch * 1e3 / ms
    # context of the device-timed step (the graph is replayed at the context the requests had reached)
    ctx_mid = main_run["mean_context"]
    step_bytes = nums["weight_bytes"] + a.batch * ctx_mid * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9

    pre_ms = prefill_run(llm, cfg, PREFILL_TOKENS, rng)
    pf = prefill_flops(cfg, a.layers, PREFILL_TOKENS)
    points = {}
    if not a.no_points:
        for b in (1, 64):
            r = decode_run(llm, cfg, b, a.context, max(8, a.steps // 2), a.warmup, rng, measure_e2e=False)
            points[f"decode_b{b}"] = round(b * 1e3 / r["ms_per_step"], 1)

    out = {
        "metric": f"decode tok/s ({shape_name}, bf16, random weights)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": shape_name, "layers": a.layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "global_batch": a.batch, "seq_len": a.context, "mean_context_timed": round(ctx_mid, 1),
                   "block_size": 16, "parallelism": "single GPU", "prefill_tokens": PREFILL_TOKENS,
                   "l2": "inputs larger than L2 (weights + cache read per step)", "peaks": pk["source"],
                   # the engine option this run sets: each decode graph in the faster of its two forms, measured at start
                   "split_norms": "auto: norms taken apart at batch sizes " + (",".join(map(str, llm.runner.split_norms_buckets())) or "none")},
        "e2e": {"value": round(a.batch * 1e3 / main_run["e2e_ms_per_step"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": main_run["h2d_bytes_per_step"],
                "d2h_bytes_per_step": main_run["d2h_bytes_per_step"],
                # the host's share of a step in us: deciding it, plan + launch, waiting for and applying the tokens
                # of the step before (one step is in flight, so the wait is where the device's time shows)
                "host_us_schedule_launch_collect": main_run.get("host_us")},
        "gpu_launches": main_run["launches_per_step"] * a.steps,
        "prefill": {"value": round(PREFILL_TOKENS * 1e3 / pre_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pre_ms, 3), "frac": round(pf / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": main_run["clocks"],
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
