#!/usr/bin/env python3
"""Kernel-level timings of the hot ops at the layer sizes of a model shape (default: Qwen3-8B).

Every op is captured back to back in one CUDA graph over operands that rotate through more memory
than the L2 holds, so that each launch reads its weights or its cache from HBM and programmatic
dependent launch overlaps neighbours as it does inside a decode step; the time per launch is the
graph's CUDA-event time divided by its launches.  Beside each time stands the time the op's bytes
(decode) or flops (prompts) take at the measured peaks.

    python bench_kernels.py                     # all sections
    python bench_kernels.py --only gemm_decode --tokens 1 8 32
    python bench_kernels.py --impl reference    # the reference's own kernels beside this package's (see below)

Sections: gemm_decode (tcgen05 swapped-operand product per split count), gemm_prompt (tcgen05 product
and the library's), attention_decode (per split count), attention_prompt, attention_short (short whole prompts, the two
tcgen05 kernels), attention_portion (a portion of a long prompt, per key split), sampling.

``--impl reference``: the same shapes and the same timing method for the reference's own CUDA kernels (norms, gate,
q/k post-processing, prompt and decode attention, small-M products, sampling), compiled unmodified for sm_100a by
``python baseline/build_ref_kernels.py /path/to/reference`` and called through their C ABI; one line per op with both
times.  Prints an ``unavailable`` line when that library has not been built.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE = dict(hidden=4096, heads=32, kv_heads=8, head_dim=128, intermediate=12288, block_size=16)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def graph_time_us(fn, launches: int, replays: int = 5) -> float:
    """fn(i) launches op number i; ``launches`` of them are captured in one graph."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(3):
            fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (replays * launches) * 1e3


def layer_products(s):
    h, H, Hkv, D, I = s["hidden"], s["heads"], s["kv_heads"], s["head_dim"], s["intermediate"]
    return [("qkv", (H + 2 * Hkv) * D, h), ("o", h, H * D), ("gate_up", 2 * I, h), ("down", h, I)]


def rotating_weights(N, K):
    copies = max(2, int(400e6 // (N * K * 2)) + 1)             # > 3 x L2 in rotation
    return [(torch.randn(N, K, device="cuda") / math.sqrt(K)).to(torch.bfloat16) for _ in range(copies)]


def gemm_decode(s, tokens_list, hbm):
    from dinfer_b200.kernels import gemm_ops as G
    print("# gemm_decode: us per launch by K splits; 'auto' is the split count the engine picks")
    for tokens in tokens_list:
        for name, N, K in layer_products(s):
            ws = rotating_weights(N, K)
            x = torch.randn(tokens, K, device="cuda").to(torch.bfloat16)
            out = torch.empty(tokens, N, dtype=torch.bfloat16, device="cuda")
            cells = []
            for splits in (1, 2, 4, 8):
                t = graph_time_us(lambda i: G.gemm_tc(x, ws[i % len(ws)], out, splits=splits), 2 * len(ws))
                cells.append(f"s{splits} {t:6.1f}")
            auto = G.decode_splits(tokens, N, K)
            t_auto = graph_time_us(lambda i: G.gemm_tc(x, ws[i % len(ws)], out), 2 * len(ws))
            ideal = N * K * 2 / hbm * 1e-3
            print(f"tokens {tokens:3d} {name:8s} N {N:6d} K {K:6d} | {' '.join(cells)} | auto s{auto} {t_auto:6.1f} us"
                  f" | weights at peak {ideal:5.1f} us -> {ideal / t_auto:.2f}", flush=True)
            del ws
    G.check_status()


def gemm_prompt(s, tokens, tflops):
    from dinfer_b200.kernels import gemm_ops as G
    print("# gemm_prompt: us per launch, this package's tcgen05 product and the library's")
    for name, N, K in layer_products(s):
        ws = rotating_weights(N, K)
        x = torch.randn(tokens, K, device="cuda").to(torch.bfloat16)
        out = torch.empty(tokens, N, dtype=torch.bfloat16, device="cuda")
        t_own = graph_time_us(lambda i: G.gemm_tc(x, ws[i % len(ws)], out), 2 * len(ws))
        t_lib = graph_time_us(lambda i: torch.mm(x, ws[i % len(ws)].t(), out=out), 2 * len(ws))
        flops = 2.0 * tokens * N * K
        print(f"tokens {tokens} {name:8s} N {N:6d} K {K:6d} | tcgen05 {t_own:7.1f} us {flops / t_own * 1e-6:7.1f} TFLOP/s"
              f" | library {t_lib:7.1f} us {flops / t_lib * 1e-6:7.1f} TFLOP/s | at peak {flops / tflops * 1e-6:6.1f} us", flush=True)
        if name == "gate_up":                                  # with the gate: one kernel against product + gate kernel
            from dinfer_b200.kernels import ops as O
            act = torch.empty(tokens, N // 2, dtype=torch.bfloat16, device="cuda")
            t_own = graph_time_us(lambda i: G.gemm_tc(x, ws[i % len(ws)], act, gated=True), 2 * len(ws))

            def lib_then_gate(i):
                torch.mm(x, ws[i % len(ws)].t(), out=out)
                O.silu_mul(out, act, pairs=True)
            t_lib = graph_time_us(lib_then_gate, 2 * len(ws))
            print(f"tokens {tokens} {name:8s} with the gate          | tcgen05 {t_own:7.1f} us (one kernel)"
                  f"      | library {t_lib:7.1f} us (product, then the gate kernel)", flush=True)
        del ws
    G.check_status()


def paged_cache(B, ctx, Hkv, D, bs, copies):
    per = (ctx + bs - 1) // bs
    caches = [torch.randn(B * per + 1, 2, Hkv, bs, D, device="cuda").to(torch.bfloat16) for _ in range(copies)]
    table = torch.randperm(B * per, device="cuda").to(torch.int32).reshape(B, per)       # scattered pages
    return caches, table


def attention_decode(s, batches, contexts, hbm):
    from dinfer_b200.kernels import attention_ops as A
    from dinfer_b200.kernels import gemm_ops as G
    H, Hkv, D, bs = s["heads"], s["kv_heads"], s["head_dim"], s["block_size"]
    print("# attention_decode: us per launch by key splits; 'auto' is the split count the engine picks")
    for B in batches:
        for ctx in contexts:
            bytes_ = B * ctx * Hkv * D * 4
            copies = min(24, max(2, int(400e6 // bytes_) + 1))
            caches, table = paged_cache(B, ctx, Hkv, D, bs, copies)
            cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
            seq = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
            q = torch.randn(B, H * D, device="cuda").to(torch.bfloat16)
            out = torch.empty(B, H * D, dtype=torch.bfloat16, device="cuda")
            cells = []
            for splits in (1, 2, 4, 8, 16):
                if splits > max(1, ctx // 64):
                    continue
                t = graph_time_us(lambda i: A.attention_decode(q, out, caches[i % copies], table, cu, seq, H, Hkv, D,
                                                               D ** -0.5, 0, splits), 2 * copies)
                cells.append(f"s{splits} {t:6.1f}")
            auto = A.decode_splits(B, Hkv, ctx)
            t_auto = graph_time_us(lambda i: A.attention_decode(q, out, caches[i % copies], table, cu, seq, H, Hkv, D,
                                                                D ** -0.5, 0, auto), 2 * copies)
            ideal = bytes_ / hbm * 1e-3
            print(f"batch {B:3d} context {ctx:5d} | {' '.join(cells)} | auto s{auto} {t_auto:6.1f} us"
                  f" | cache at peak {ideal:6.1f} us -> {ideal / t_auto:.2f}", flush=True)
            del caches
    G.check_status()


def attention_prompt(s, tokens_list, tflops):
    from dinfer_b200.kernels import attention_ops as A
    from dinfer_b200.kernels import gemm_ops as G
    H, Hkv, D, bs = s["heads"], s["kv_heads"], s["head_dim"], s["block_size"]
    print("# attention_prompt: one request, whole prompt in one step (causal), us per launch")
    for T in tokens_list:
        caches, table = paged_cache(1, T, Hkv, D, bs, 4)
        cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
        seq = torch.tensor([T], dtype=torch.int32, device="cuda")
        qkv = torch.randn(T, (H + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
        q = qkv[:, :H * D]
        out = torch.empty(T, H * D, dtype=torch.bfloat16, device="cuda")
        flops = 4.0 * (T * (T + 1) / 2) * D * H
        t_umma = graph_time_us(lambda i: A.attention_umma(q, out, caches[i % 4], table, cu, seq, H, Hkv, D, D ** -0.5,
                                                          0, T), 8)
        t_tc = graph_time_us(lambda i: A.attention_tc(q, out, caches[i % 4], table, cu, seq, H, Hkv, D, D ** -0.5,
                                                      0, T, False, True, 1), 8)
        print(f"tokens {T:5d} | tcgen05 {t_umma:7.1f} us {flops / t_umma * 1e-6:6.1f} TFLOP/s"
              f" | mma.sync {t_tc:7.1f} us {flops / t_tc * 1e-6:6.1f} TFLOP/s | at peak {flops / tflops * 1e-6:6.1f} us", flush=True)
        del caches
    G.check_status()


def attention_short(s):
    """Whole short prompts, as a serving step takes them in: the two tcgen05 kernels beside each other."""
    from dinfer_b200.kernels import attention_ops as A
    from dinfer_b200.kernels import gemm_ops as G
    H, Hkv, D, bs = s["heads"], s["kv_heads"], s["head_dim"], s["block_size"]
    print(f"# attention_short: B whole prompts of P tokens in one step, us per launch; the engine takes the 64-key kernel up to "
          f"{A.UMMA_SHORT_CONTEXT} tokens")
    for B, P in ((1, 32), (1, 128), (8, 128), (32, 128), (1, 512), (4, 512), (1, 1024)):
        caches, table = paged_cache(B, P, Hkv, D, bs, 4)
        cu = torch.arange(0, (B + 1) * P, P, dtype=torch.int32, device="cuda")
        seq = torch.full((B,), P, dtype=torch.int32, device="cuda")
        qkv = torch.randn(B * P, (H + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
        q = qkv[:, :H * D]
        out = torch.empty(B * P, H * D, dtype=torch.bfloat16, device="cuda")
        bound = A.umma_pair_bound([P] * B, H // Hkv)
        ks = A.umma_key_splits([P] * B, H // Hkv, Hkv, D, P)
        t128 = graph_time_us(lambda i: A.attention_umma(q, out, caches[i % 4], table, cu, seq, H, Hkv, D, D ** -0.5,
                                                        0, P, ks, bound), 8)
        t64 = graph_time_us(lambda i: A.attention_umma64(q, out, caches[i % 4], table, cu, seq, H, Hkv, D, D ** -0.5,
                                                         0, P, bound), 8)
        print(f"prompts {B:3d} tokens {P:5d} | 64-key tiles {t64:6.1f} us | 128-key tiles {t128:6.1f} us", flush=True)
        del caches
    G.check_status()


def attention_portion(s, tflops):
    """The tcgen05 prompt attention on one portion of a long prompt (chunked prefill): few row tiles, long histories."""
    from dinfer_b200.kernels import attention_ops as A
    from dinfer_b200.kernels import gemm_ops as G
    H, Hkv, D, bs = s["heads"], s["kv_heads"], s["head_dim"], s["block_size"]
    print("# attention_portion: a portion behind a history, us per launch by the CTAs that share a row-tile pair's keys;"
          " 'auto' is the engine's choice")
    for P, C in ((512, 4096), (512, 16384), (256, 8192), (128, 4096), (1024, 8192)):
        caches, table = paged_cache(1, C, Hkv, D, bs, 4)
        cu = torch.tensor([0, P], dtype=torch.int32, device="cuda")
        seq = torch.tensor([C], dtype=torch.int32, device="cuda")
        qkv = torch.randn(P, (H + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
        q = qkv[:, :H * D]
        out = torch.empty(P, H * D, dtype=torch.bfloat16, device="cuda")
        flops = 4.0 * (P * (C - P) + P * (P + 1) / 2) * D * H
        auto = A.umma_key_splits([P], H // Hkv, Hkv, D, C)
        cells = []
        for ks in (1, 2, 4, 8):
            t = graph_time_us(lambda i: A.attention_umma(q, out, caches[i % 4], table, cu, seq, H, Hkv, D, D ** -0.5,
                                                         0, P, ks), 8)
            cells.append(f"s{ks} {t:6.1f}")
            if ks == auto:
                t_auto = t
        print(f"portion {P:5d} context {C:6d} | {' '.join(cells)} | auto s{auto} {t_auto:6.1f} us "
              f"{flops / t_auto * 1e-6:6.1f} TFLOP/s | at peak {flops / tflops * 1e-6:6.1f} us", flush=True)
        del caches
    G.check_status()


def sampling(vocab, rows_list):
    """The sampling kernels behind a step: device time per launch (the rows' columns already on the device)."""
    from dinfer_b200.sampling import sampler as S
    print("# sampling: us per launch over f32 logits [rows, vocabulary], by what the rows ask for")
    for R in rows_list:
        logits = torch.randn(R, vocab, device="cuda") * 3
        out = torch.empty(R, dtype=torch.int32, device="cuda")
        temp = torch.full((R,), 0.7, device="cuda")
        seeds = torch.arange(R, dtype=torch.int64, device="cuda")
        offs = torch.full((R,), 3, dtype=torch.int64, device="cuda")
        one = torch.ones(R, device="cuda")
        zero = torch.zeros(R, device="cuda")

        def ints(v):
            return torch.full((R,), v, dtype=torch.int32, device="cuda")
        cases = [("greedy", lambda i: S.argmax(logits, out)),
                 ("temperature", lambda i: S.sample(logits, temp, seeds, offs, ints(-1), one, zero, out)),
                 ("top-k 20 + top-p 0.95", lambda i: S.sample(logits, temp, seeds, offs, ints(20), one * 0.95, zero, out)),
                 ("top-p 0.95 alone", lambda i: S.sample(logits, temp, seeds, offs, ints(-1), one * 0.95, zero, out)),
                 ("top-k 1000 (radix descent)", lambda i: S.sample(logits, temp, seeds, offs, ints(1000), one, zero, out))]
        cells = [f"{name} {graph_time_us(fn, 8):6.1f}" for name, fn in cases]
        print(f"rows {R:3d} | " + " | ".join(cells), flush=True)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--only", choices=["gemm_decode", "gemm_prompt", "attention_decode", "attention_prompt", "attention_short", "attention_portion", "sampling",
                                       "small_ops"])
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours",
                    help="reference: time the reference's own kernels beside this package's")
    ap.add_argument("--tokens", type=int, nargs="*", default=[1, 8, 32], help="rows of the decode products")
    ap.add_argument("--batches", type=int, nargs="*", default=[1, 8, 64], help="requests of the decode attention")
    ap.add_argument("--contexts", type=int, nargs="*", default=[1024, 4096, 16384])
    ap.add_argument("--prompt-tokens", type=int, nargs="*", default=[2048, 8192])
    ap.add_argument("--heads", type=int, nargs=3, metavar=("H", "HKV", "D"), default=None,
                    help="attention sections: other head counts and head size than the Qwen3-8B shape's 32 8 128")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        print("bench_kernels.py needs a GPU", file=sys.stderr)
        return 2
    hbm, tflops, source = peaks()
    print(f"# peaks ({source}): {hbm:.1f} GB/s, {tflops:.1f} TFLOP/s bf16; {torch.cuda.get_device_name(0)}")
    torch.manual_seed(0)
    if a.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import ref_kernels
        return ref_kernels.run(sys.modules[__name__], a, hbm, tflops)
    if a.heads:
        SHAPE.update(heads=a.heads[0], kv_heads=a.heads[1], head_dim=a.heads[2])
        print(f"# heads {a.heads[0]}, kv heads {a.heads[1]}, head size {a.heads[2]}")
    todo = [a.only] if a.only else ["gemm_decode", "gemm_prompt", "attention_decode", "attention_prompt", "attention_short", "attention_portion", "sampling"]
    if "gemm_decode" in todo:
        gemm_decode(SHAPE, a.tokens, hbm)
    if "gemm_prompt" in todo:
        gemm_prompt(SHAPE, a.prompt_tokens[0], tflops)
    if "attention_decode" in todo:
        attention_decode(SHAPE, a.batches, a.contexts, hbm)
    if "attention_prompt" in todo:
        attention_prompt(SHAPE, a.prompt_tokens, tflops)
    if "attention_short" in todo:
        attention_short(SHAPE)
    if "attention_portion" in todo:
        attention_portion(SHAPE, tflops)
    if "sampling" in todo:
        sampling(151936, a.batches)
    return 0


if __name__ == "__main__":
    sys.exit(main())
