#!/usr/bin/env python3
"""Makes tests/golden/ref_ops.npz: small inputs and what the reference's OWN torch-CPU formulas make of them
(rayze-ai/dinfer, scripts/verify/ops_parity_ref.py).  The reference's Rust/CUDA model cannot be built on a machine
without cargo and a GPU, so these per-part formulas are the only code of the reference that runs here; the
whole-model path of tests/plain_model.py (layer order, final norm, tied head) rests on the formulas it cites.

Taken from the reference, by executing its definitions:
  rmsnorm :59-61, rope_neox :123-128, attn_ref :208-222              their outputs
  chk_fused_add_rmsnorm :70-76, chk_silu_mul :84-89, chk_qkv_post :131-152
      the reference's checks of its kernels' outputs.  Each is handed the plain implementation's result as the
      "kernel output"; what the check itself computes as expected (the `want` it passes to its `close`) is
      recorded, together with the check's own verdict on the plain implementation's result
  penalties_ref :285-299, topk_topp_ref :301-312                     their outputs

Run once with the reference checked out:  python tests/golden/make_golden.py /path/to/reference
Only definitions of the reference file are executed (its command-line part is not).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_model as P  # noqa: E402


def load_reference(ref_root: str) -> dict:
    path = os.path.join(ref_root, "scripts", "verify", "ops_parity_ref.py")
    text = open(path, encoding="utf-8").read()
    cut = text.index("def chk_rmsnorm")
    ns = {"__name__": "ref_ops"}
    saved = sys.argv
    sys.argv = [path]
    try:
        exec(compile(text[:cut], path, "exec"), ns)
        rest = text[cut:]
        for fn in ("chk_fused_add_rmsnorm", "chk_silu_mul", "rope_neox", "chk_qkv_post", "attn_ref", "penalties_ref",
                   "topk_topp_ref"):
            a = rest.index(f"def {fn}(")
            b = rest.index("\n\n\n", a)
            exec(compile(rest[a:b], path, "exec"), ns)
    finally:
        sys.argv = saved
    return ns


def run_check(ns: dict, name: str, t: dict, meta: dict):
    """Run one of the reference's checks; returns (what it computed as expected, in the order of its `close`
    calls; its verdict)."""
    wants = []
    inner = ns["close"]

    def close(got, want, atol, rtol):
        wants.append(want.clone().float())
        return inner(got, want, atol, rtol)

    ns["close"] = close
    ns["ROWS"].clear()
    try:
        ns[name](t, meta, "golden")
    finally:
        ns["close"] = inner
    (_, _, err, note, ok), = ns["ROWS"]
    return wants, bool(ok), float(err)


def main(ref_root: str) -> None:
    ns = load_reference(ref_root)
    bf = ns["bf"]
    g = torch.Generator().manual_seed(11)
    out = {}
    x = torch.randn(5, 96, generator=g)
    w = 1 + 0.2 * torch.randn(96, generator=g)
    out["norm_x"], out["norm_w"], out["norm_eps"] = x, w, torch.tensor(1e-5)
    out["norm_y"] = ns["rmsnorm"](x, w, 1e-5)
    T, H, HK, D, hist = 6, 6, 2, 32, 9
    q = torch.randn(T, H, D, generator=g)
    k = torch.randn(hist + T, HK, D, generator=g)
    v = torch.randn(hist + T, HK, D, generator=g)
    out["attn_q"], out["attn_k"], out["attn_v"] = q, k, v
    out["attn_hist"], out["attn_scale"] = torch.tensor(hist), torch.tensor(D ** -0.5)
    out["attn_o"] = ns["attn_ref"](q, k, v, hist, D ** -0.5)
    pos = torch.tensor([0, 1, 5, 77, 200])
    half = D // 2
    inv = 1.0 / (1e6 ** (2.0 * torch.arange(half, dtype=torch.float64) / D))
    ang = pos.to(torch.float64)[:, None] * inv[None, :]
    cs = torch.cat([ang.cos(), ang.sin()], 1).float()
    xr = torch.randn(5, 3, D, generator=g)
    out["rope_x"], out["rope_pos"], out["rope_theta"] = xr, pos, torch.tensor(1e6)
    out["rope_y"] = ns["rope_neox"](xr, cs[:, None, :])

    # ---- the fused residual add and norm (inputs in the storage type, as the kernel gets them)
    xa, ra = bf(torch.randn(7, 96, generator=g)), bf(torch.randn(7, 96, generator=g) * 3)
    wa = bf(1 + 0.2 * torch.randn(96, generator=g))
    res, normed = P.add_and_norm(ra.double(), xa.double(), wa.double(), 1e-5)
    wants, ok, err = run_check(ns, "chk_fused_add_rmsnorm",
                               {"x": xa, "res_in": ra, "w": wa, "res_out": bf(res.float()), "out": bf(normed.float())},
                               {"eps": 1e-5})
    assert ok, ("the reference's check rejects the plain add + norm", err)
    out["addnorm_x"], out["addnorm_res"], out["addnorm_w"] = xa, ra, wa
    out["addnorm_res_out"], out["addnorm_out"] = wants

    # ---- the gate (silu(first half) * second half)
    gu = bf(torch.randn(5, 2 * 56, generator=g) * 2)
    wants, ok, err = run_check(ns, "chk_silu_mul", {"x": gu, "out": bf(P.gate(gu.double()).float())}, {})
    assert ok, ("the reference's check rejects the plain gate", err)
    out["gate_x"], (out["gate_out"],) = gu, wants

    # ---- q/k head norm, then rotation, v untouched, and what goes into the cache
    T, H, HK, D, bs, theta, maxpos = 9, 6, 2, 32, 4, 1e6, 64
    qkv = bf(torch.randn(T, (H + 2 * HK) * D, generator=g))
    wq, wk = bf(1 + 0.2 * torch.randn(D, generator=g)), bf(1 + 0.2 * torch.randn(D, generator=g))
    pos = torch.tensor([0, 1, 2, 17, 18, 40, 41, 42, 63])
    slots = torch.tensor([4, 5, 6, -1, 20, 33, 34, 35, 9])              # one token without a slot
    inv = 1.0 / (theta ** (2.0 * torch.arange(D // 2, dtype=torch.float64) / D))
    ang = torch.arange(maxpos, dtype=torch.float64)[:, None] * inv[None, :]
    table = torch.cat([ang.cos(), ang.sin()], 1).float()                # [max positions, D] = cos | sin, as nn.rs:157-173
    rows, kv = P.qk_post(qkv.double(), pos, H, HK, D, wq.double(), wk.double(), 1e-5, theta)
    cache = torch.zeros(40, HK, 2, D)                                   # the reference's layout [slot, kv head, k|v, D]
    for i in range(T):
        if int(slots[i]) >= 0:
            cache[int(slots[i])] = bf(kv[i].float())
    wants, ok, err = run_check(ns, "chk_qkv_post",
                               {"qkv_in": qkv, "cos_sin": table, "pos": pos, "wq": wq, "wk": wk, "slots": slots,
                                "qkv_out": bf(rows.float()), "cache": cache},
                               {"heads": H, "kv_heads": HK, "head_dim": D, "eps": 1e-5, "block_size": bs})
    assert ok, ("the reference's check rejects the plain q/k post-processing", err)
    out["qkpost_qkv"], out["qkpost_wq"], out["qkpost_wk"], out["qkpost_pos"] = qkv, wq, wk, pos
    out["qkpost_slots"], out["qkpost_theta"] = slots, torch.tensor(theta)
    out["qkpost_dims"] = torch.tensor([H, HK, D])
    out["qkpost_rows"], out["qkpost_cache"] = wants

    # ---- penalties and the top-k / top-p filter
    V = 40
    logits = torch.randn(3, V, generator=g) * 3
    ids = torch.tensor([3, 30, 30, 7, 30, 3, 11,   1, 2, 2,   5, 5, 5, 6], dtype=torch.int32)
    offs, plen = [0, 7, 10, 14], [2, 3, 1]
    rep, freq, pres = [1.5, 1.0, 0.8], [0.3, 0.0, 0.25], [0.2, 0.0, 0.1]
    out["pen_logits"], out["pen_ids"] = logits, ids
    out["pen_offsets"], out["pen_prompt_len"] = torch.tensor(offs), torch.tensor(plen)
    out["pen_rep"], out["pen_freq"], out["pen_pres"] = torch.tensor(rep), torch.tensor(freq), torch.tensor(pres)
    out["pen_out"] = ns["penalties_ref"](logits, ids, offs, plen, rep, freq, pres)
    row = torch.randn(60, generator=g) * 2.5
    cases = [(5, 1.0), (0, 0.7), (8, 0.5), (60, 0.9), (1, 0.3), (0, 1.0), (12, 0.95)]
    out["filter_row"] = row
    out["filter_cases"] = torch.tensor(cases, dtype=torch.float64)
    out["filter_out"] = torch.stack([ns["topk_topp_ref"](row, kk, pp) for kk, pp in cases])

    dst = os.path.join(HERE, "ref_ops.npz")
    np.savez(dst, **{k: v.numpy() for k, v in out.items()})
    print("wrote", dst, {k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
