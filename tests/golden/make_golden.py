#!/usr/bin/env python3
"""Makes tests/golden/ref_ops.npz: small inputs and the outputs of the reference's OWN torch-CPU
formulas for them (rayze-ai/dinfer, scripts/verify/ops_parity_ref.py: rmsnorm :59-61, rope_neox
:123-128, attn_ref :208-222).  The reference's Rust/CUDA model cannot be built on a machine
without cargo and a GPU, so these per-part formulas are the only code of the reference that runs
here; the whole-model path of tests/plain_model.py rests on the formulas it cites.

Run once with the reference checked out:  python tests/golden/make_golden.py /path/to/reference
Only the function definitions of the reference file are executed (the text above its main part).
"""
import os
import sys

import numpy as np
import torch


def main(ref_root: str) -> None:
    path = os.path.join(ref_root, "scripts", "verify", "ops_parity_ref.py")
    text = open(path, encoding="utf-8").read()
    cut = text.index("def chk_rmsnorm")
    head = text[:cut]
    ns = {"__name__": "ref_ops"}
    saved = sys.argv
    sys.argv = [path]
    try:
        exec(compile(head, path, "exec"), ns)
        rest = text[cut:]
        for fn in ("rope_neox", "attn_ref"):
            a = rest.index(f"def {fn}(")
            b = rest.index("\n\n\n", a)
            exec(compile(rest[a:b], path, "exec"), ns)
    finally:
        sys.argv = saved
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
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_ops.npz")
    np.savez(dst, **{k: v.numpy() for k, v in out.items()})
    print("wrote", dst, {k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
