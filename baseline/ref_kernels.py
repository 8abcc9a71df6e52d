"""The kernel-level reference arm of ``bench_kernels.py``: the reference's own Qwen3-path kernels, compiled unmodified
for sm_100a by ``baseline/build_ref_kernels.py`` and called through their stock C ABI
(crates/kernels/cuda/kernels.h), timed at the same shapes and by the same method as this package's kernels (one
CUDA graph of launches over operands that rotate through more than the L2 holds).

How the reference would run each op on a B200, as its engine does:
  * decode products (at most 32 rows): its tuner times its two small-M kernels over their candidate grids
    (crates/kernels/src/arch.rs:149-157: K splits by wave targets, 4 or 8 warps, 1/2/4 stripes) and cuBLASLt and keeps
    the fastest (crates/kernels/src/gemm.rs:1148-1262); here the same candidates are timed and the fastest is
    reported, with ``torch.mm`` standing for cuBLASLt;
  * decode attention: ``gqa_decode_bf16``, which picks its own splits and forwards to the v3 kernel and the merge
    (crates/kernels/cuda/gqa.cu:1727-1812);
  * prompt attention: ``gqa_prefill_bf16`` over the step's own k/v rows for a whole prompt, ``gqa_paged_bf16`` over
    the cache for a portion with history (models/qwen3/src/model.rs:232-311);
  * q/k post-processing, norms (thread layout 2 = 1024 threads a row for this width: crates/kernels/src/arch.rs:206-220),
    the gate, argmax and sampling: their one entry point each.
The reference's cache is ``[blocks, block_size, kv_heads, 2, head_dim]`` (models/qwen3/src/model.rs:20-25); it is
filled in that layout, the kernels are not adapted.
"""
from __future__ import annotations

import ctypes
import math
import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libdinfer_ref_kernels.so")


def load():
    if not os.path.isfile(LIB_PATH):
        raise FileNotFoundError(f"{LIB_PATH} is not built: run python baseline/build_ref_kernels.py /path/to/reference")
    return ctypes.CDLL(LIB_PATH)


def _p(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ok(rc, what):
    if rc != 0:
        raise RuntimeError(f"reference {what} returned {rc}")


def eager_time_us(fn, reps: int = 20) -> float:
    """For entry points that copy a host variable to the device at every call (not capturable): launched one by
    one, timed with CUDA events; only used for kernels long enough that the launch gap does not show."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def gemm_decode(lib, K_, s, tokens_list, hbm):
    from dinfer_b200.kernels import gemm_ops as G
    mma, simt = lib.gemm_small_m_mma_bf16, lib.gemm_small_m_bf16
    mma.argtypes = [c_void_p] * 6 + [c_int64] * 6 + [c_void_p]
    simt.argtypes = [c_void_p] * 5 + [c_int64] * 4 + [c_void_p]
    print("# gemm_decode: us per launch; reference = the fastest of its small-M kernels' candidates and the library")
    for tokens in tokens_list:
        for name, N, K in K_.layer_products(s):
            ws = K_.rotating_weights(N, K)
            x = torch.randn(tokens, K, device="cuda").to(torch.bfloat16)
            out = torch.empty(tokens, N, dtype=torch.bfloat16, device="cuda")
            partial = torch.empty(16 * tokens * N, dtype=torch.float32, device="cuda")
            counters = torch.zeros((N + 7) // 8 + 8, dtype=torch.int32, device="cuda")
            n = 2 * len(ws)
            best = (float("inf"), "")
            for splits in (1, 2, 4, 8, 16):
                for warps in (4, 8):
                    for stripes in (1, 2, 4):
                        def f(i):
                            _ok(mma(_p(x), _p(ws[i % len(ws)]), None, _p(out), _p(partial), _p(counters), tokens, N, K,
                                    splits, warps, stripes, _stream()), "gemm_small_m_mma_bf16")
                        t = K_.graph_time_us(f, n, replays=3)
                        best = min(best, (t, f"mma(s{splits}w{warps}r{stripes})"))
            for splits in (1, 2, 4, 8):
                def f(i):
                    _ok(simt(_p(x), _p(ws[i % len(ws)]), None, _p(out), _p(partial), tokens, N, K, splits, _stream()),
                        "gemm_small_m_bf16")
                t = K_.graph_time_us(f, n, replays=3)
                best = min(best, (t, f"small_m(s{splits})"))
            t = K_.graph_time_us(lambda i: torch.mm(x, ws[i % len(ws)].t(), out=out), n, replays=3)
            best = min(best, (t, "library"))
            t_own = K_.graph_time_us(lambda i: G.gemm_tc(x, ws[i % len(ws)], out), n)
            ideal = N * K * 2 / hbm * 1e-3
            print(f"tokens {tokens:3d} {name:8s} N {N:6d} K {K:6d} | reference {best[0]:6.1f} us {best[1]:16s} | ours {t_own:6.1f} us"
                  f" | x{best[0] / t_own:.2f} | weights at peak {ideal:5.1f} us", flush=True)
            del ws


def attention_decode(lib, K_, s, batches, contexts, hbm):
    from dinfer_b200.kernels import attention_ops as A
    H, Hkv, D, bs = s["heads"], s["kv_heads"], s["head_dim"], s["block_size"]
    fn = lib.gqa_decode_bf16
    fn.argtypes = [c_void_p] * 6 + [c_int64] * 6 + [c_float, c_int64, c_void_p, c_void_p]
    v3, merge = lib.gqa_decode_v3_bf16, lib.gqa_decode_merge_v2_launch
    v3.argtypes = [c_void_p] * 7 + [c_int64] * 6 + [c_float, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]
    merge.argtypes = [c_void_p] * 4 + [c_int] * 5 + [c_void_p]
    group = H // Hkv
    print("# attention_decode: us per launch.  reference: its stock entry gqa_decode_bf16 for groups of up to 2 (which it "
          "takes to its v3 kernel + merge); for a group of 4 its v3 kernel + merge called directly with the stock "
          "entry's split rule")
    for B in batches:
        for ctx in contexts:
            bytes_ = B * ctx * Hkv * D * 4
            copies = min(24, max(2, int(400e6 // bytes_) + 1))
            caches, table = K_.paged_cache(B, ctx, Hkv, D, bs, copies)                 # ours: [blocks, 2, Hkv, bs, D]
            ref_caches = [c.reshape(c.shape[0], bs, Hkv, 2, D) for c in caches]        # the same bytes as [blocks, bs, Hkv, 2, D]
            cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
            seq = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
            q = torch.randn(B, H * D, device="cuda").to(torch.bfloat16)
            out = torch.empty(B, H * D, dtype=torch.bfloat16, device="cuda")
            scratch = torch.empty(B * H * 32 * (D + 2), dtype=torch.float32, device="cuda")

            # The stock entry sends a group above 2 to the reference's first decode kernel (gqa.cu:1753,1796-1806).
            # With a group of 4 at batch 64, context 1024, that path raised an illegal memory access on a B200 here;
            # reading the kernel did not show why, so it is not run: the v3 kernel, which takes a group of 4 when
            # called directly, stands for the reference at such shapes.
            if group <= 2:
                def ref(i):
                    _ok(fn(_p(q), _p(ref_caches[i % copies]), _p(table), _p(seq), _p(out), _p(scratch), B, H, Hkv, D, bs,
                           table.shape[1], D ** -0.5, H * D, _p(cu), _stream()), "gqa_decode_bf16")
                how = "stock entry"
            elif group == 4:
                splits = max(1, min(32, (2048 + B * Hkv - 1) // (B * Hkv)))               # gqa.cu:1756-1757

                def ref(i):
                    _ok(v3(_p(q), _p(ref_caches[i % copies]), _p(table), _p(seq), _p(cu), _p(scratch),
                           _p(out) if splits == 1 else None, B, H, Hkv, D, bs, table.shape[1], D ** -0.5, H * D, splits, 32,
                           0, 0, _stream()), "gqa_decode_v3_bf16")
                    if splits > 1:
                        _ok(merge(_p(scratch), _p(cu), _p(seq), _p(out), B, H, D, splits, 32, _stream()), "gqa_decode_merge_v2")
                how = f"v3 direct, {splits} splits"
            else:
                print(f"batch {B:3d} context {ctx:5d} | reference: no decode kernel of its own is timed for a group of {group}")
                continue
            t_ref = K_.graph_time_us(ref, 2 * copies)
            auto = A.decode_splits(B, Hkv, ctx)
            t_own = K_.graph_time_us(lambda i: A.attention_decode(q, out, caches[i % copies], table, cu, seq, H, Hkv, D,
                                                                  D ** -0.5, 0, auto), 2 * copies)
            ideal = bytes_ / hbm * 1e-3
            print(f"batch {B:3d} context {ctx:5d} | reference {t_ref:7.1f} us ({how}) | ours {t_own:7.1f} us | x{t_ref / t_own:.2f}"
                  f" | cache at peak {ideal:6.1f} us", flush=True)
            del caches, ref_caches


def attention_prompt(lib, K_, s, tokens_list, tflops):
    from dinfer_b200.kernels import attention_ops as A
    H, Hkv, D, bs = s["heads"], s["kv_heads"], s["head_dim"], s["block_size"]
    pre, paged = lib.gqa_prefill_bf16, lib.gqa_paged_bf16
    pre.argtypes = [c_void_p] * 5 + [c_int64] * 5 + [c_float, c_int64, c_int64, c_int, c_void_p]
    paged.argtypes = [c_void_p] * 6 + [c_int64] * 7 + [c_float, c_int64, c_int, c_int, c_void_p]
    print("# attention_prompt: one request, whole prompt in one step (causal), us per launch, launched one by one")
    for T in tokens_list:
        caches, table = K_.paged_cache(1, T, Hkv, D, bs, 4)
        ref_caches = [c.reshape(c.shape[0], bs, Hkv, 2, D) for c in caches]
        cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
        seq = torch.tensor([T], dtype=torch.int32, device="cuda")
        qkv = torch.randn(T, (H + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
        q, k, v = qkv[:, :H * D], qkv[:, H * D:(H + Hkv) * D], qkv[:, (H + Hkv) * D:]
        out = torch.empty(T, H * D, dtype=torch.bfloat16, device="cuda")
        flops = 4.0 * (T * (T + 1) / 2) * D * H
        stride = qkv.stride(0)

        def ref_rows(i):
            _ok(pre(_p(q), _p(k), _p(v), _p(out), _p(cu), 1, T, H, Hkv, D, D ** -0.5, stride, stride, 0, _stream()),
                "gqa_prefill_bf16")

        def ref_paged(i):
            _ok(paged(_p(q), _p(ref_caches[i % 4]), _p(table), _p(seq), _p(cu), _p(out), 1, T, H, Hkv, D, bs, table.shape[1],
                      D ** -0.5, stride, 0, 0, _stream()), "gqa_paged_bf16")
        t_rows, t_paged = eager_time_us(ref_rows), eager_time_us(ref_paged)
        t_own = eager_time_us(lambda i: A.attention_umma(q, out, caches[i % 4], table, cu, seq, H, Hkv, D, D ** -0.5, 0, T))
        print(f"tokens {T:5d} | reference {t_rows:7.1f} us over the step's rows, {t_paged:7.1f} us over the cache"
              f" ({flops / t_paged * 1e-6:5.1f} TFLOP/s) | ours {t_own:7.1f} us ({flops / t_own * 1e-6:6.1f} TFLOP/s)"
              f" | x{t_paged / t_own:.2f} | at peak {flops / tflops * 1e-6:6.1f} us", flush=True)
        del caches, ref_caches


def small_ops(lib, K_, s, rows_list, hbm):
    from dinfer_b200.kernels import ops as O
    from dinfer_b200.parts.rope import rope_table
    h, H, Hkv, D, I, bs = s["hidden"], s["heads"], s["kv_heads"], s["head_dim"], s["intermediate"], s["block_size"]
    post = lib.qkv_post_bf16
    post.argtypes = [c_void_p] * 7 + [c_int64] * 4 + [c_float, c_int64, c_void_p]
    addnorm = lib.fused_add_rmsnorm_bf16
    addnorm.argtypes = [c_void_p] * 4 + [c_int64, c_int64, c_float, c_int, c_int, c_void_p]
    gate = lib.silu_and_mul_bf16
    gate.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_void_p]
    print("# q/k post-processing, residual add + norm, gate: us per launch")
    maxpos = 8192
    table = rope_table(D, 1e6, maxpos, "cuda")                                  # [max positions, D] f32 = cos | sin
    for T in rows_list:
        nb = max(T // bs + 2, 64)
        copies = max(2, min(16, int(300e6 // max(1, T * (H + 2 * Hkv) * D * 2))))
        qkvs = [torch.randn(T, (H + 2 * Hkv) * D, device="cuda").to(torch.bfloat16) for _ in range(copies)]
        wq = torch.ones(D, dtype=torch.bfloat16, device="cuda")
        pos = torch.arange(T, dtype=torch.int32, device="cuda") % maxpos
        slots32 = torch.randperm(nb * bs, device="cuda")[:T].to(torch.int32)
        slots64 = slots32.to(torch.int64)
        cache = torch.zeros(nb, 2, Hkv, bs, D, dtype=torch.bfloat16, device="cuda")
        ref_cache = cache.reshape(nb, bs, Hkv, 2, D)
        t_ref = K_.graph_time_us(lambda i: _ok(post(_p(qkvs[i % copies]), _p(wq), _p(wq), _p(pos), _p(table), _p(ref_cache),
                                                    _p(slots64), T, H, Hkv, D, 1e-6, bs, _stream()), "qkv_post_bf16"), 2 * copies)
        t_own = K_.graph_time_us(lambda i: O.qk_post(qkvs[i % copies], pos, H, Hkv, D, 1e-6, wq, wq, table, cache, slots32, bs),
                                 2 * copies)
        print(f"rows {T:5d} q/k norm + rotation + cache write | reference {t_ref:6.1f} us | ours {t_own:6.1f} us | x{t_ref / t_own:.2f}",
              flush=True)
        del qkvs
        copies = max(2, min(16, int(300e6 // max(1, T * h * 2))))
        xs = [torch.randn(T, h, device="cuda").to(torch.bfloat16) for _ in range(copies)]
        res16 = torch.randn(T, h, device="cuda").to(torch.bfloat16)
        res32 = res16.float()
        w = torch.ones(h, dtype=torch.bfloat16, device="cuda")
        o = torch.empty(T, h, dtype=torch.bfloat16, device="cuda")
        t_ref = K_.graph_time_us(lambda i: _ok(addnorm(_p(xs[i % copies]), _p(res16), _p(w), _p(o), T, h, 1e-6, 2, 0, _stream()),
                                               "fused_add_rmsnorm_bf16"), 2 * copies)
        t_own = K_.graph_time_us(lambda i: O.rmsnorm(res32, w, 1e-6, delta=xs[i % copies], out=o), 2 * copies)
        print(f"rows {T:5d} residual add + norm (ours keeps the residual in f32: 4 more bytes a value each way) | reference {t_ref:6.1f} us"
              f" | ours {t_own:6.1f} us | x{t_ref / t_own:.2f}", flush=True)
        del xs
        copies = max(2, min(16, int(300e6 // max(1, T * 2 * I * 2))))
        gus = [torch.randn(T, 2 * I, device="cuda").to(torch.bfloat16) for _ in range(copies)]
        act = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
        t_ref = K_.graph_time_us(lambda i: _ok(gate(_p(gus[i % copies]), _p(act), T, I, _stream()), "silu_and_mul_bf16"), 2 * copies)
        t_own = K_.graph_time_us(lambda i: O.silu_mul(gus[i % copies], act), 2 * copies)
        print(f"rows {T:5d} gate (the engine's own path has it inside the product's epilogue) | reference {t_ref:6.1f} us"
              f" | ours {t_own:6.1f} us | x{t_ref / t_own:.2f}", flush=True)
        del gus


def sampling(lib, K_, vocab, rows_list):
    from dinfer_b200.sampling import sampler as S
    am, sm = lib.argmax_f32, lib.sample_f32
    am.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_void_p]
    sm.argtypes = [c_void_p] * 5 + [c_int64, c_int64, c_void_p]
    print("# sampling over f32 logits [rows, vocabulary]: us per launch")
    for R in rows_list:
        logits = torch.randn(R, vocab, device="cuda") * 3
        out = torch.empty(R, dtype=torch.int32, device="cuda")
        temp = torch.full((R,), 0.7, device="cuda")
        seeds = torch.arange(R, dtype=torch.int64, device="cuda")
        offs = torch.full((R,), 3, dtype=torch.int64, device="cuda")
        one, zero = torch.ones(R, device="cuda"), torch.zeros(R, device="cuda")
        k_off = torch.full((R,), -1, dtype=torch.int32, device="cuda")
        t_ra = K_.graph_time_us(lambda i: _ok(am(_p(logits), _p(out), R, vocab, _stream()), "argmax_f32"), 8)
        t_oa = K_.graph_time_us(lambda i: S.argmax(logits, out), 8)
        t_rs = K_.graph_time_us(lambda i: _ok(sm(_p(logits), _p(temp), _p(seeds), _p(offs), _p(out), R, vocab, _stream()),
                                              "sample_f32"), 8)
        t_os = K_.graph_time_us(lambda i: S.sample(logits, temp, seeds, offs, k_off, one, zero, out), 8)
        print(f"rows {R:3d} | greedy: reference {t_ra:6.1f} us, ours {t_oa:6.1f} us, x{t_ra / t_oa:.2f}"
              f" | temperature: reference {t_rs:6.1f} us, ours {t_os:6.1f} us, x{t_rs / t_os:.2f}", flush=True)


def run(K_, a, hbm, tflops) -> int:
    """``K_``: the bench_kernels module (its timing method, shapes and operand makers)."""
    try:
        lib = load()
    except (FileNotFoundError, OSError) as e:
        print(f'{{"impl": "reference", "unavailable": "{e}"}}')
        return 0
    s = K_.SHAPE
    todo = [a.only] if a.only else ["gemm_decode", "attention_decode", "attention_prompt", "small_ops", "sampling"]
    if "gemm_decode" in todo:
        gemm_decode(lib, K_, s, a.tokens, hbm)
    if "attention_decode" in todo:
        attention_decode(lib, K_, s, a.batches, a.contexts, hbm)
    if "attention_prompt" in todo:
        attention_prompt(lib, K_, s, a.prompt_tokens, tflops)
    if "small_ops" in todo:
        small_ops(lib, K_, s, [8, 2048], hbm)
    if "sampling" in todo:
        sampling(lib, K_, 151936, a.batches)
    if "gemm_prompt" in todo:
        print("# gemm_prompt: the reference calls cuBLASLt for prompt products (crates/kernels/src/gemm.rs:649-690); "
              "the 'library' column of the default run is that product")
    return 0
