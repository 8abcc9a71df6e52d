"""The plain implementation against the reference's own torch-CPU formulas (outputs committed under
tests/golden/, made by tests/golden/make_golden.py) and against itself (no GPU)."""
import os

import numpy as np
import torch

import helpers as H
import plain_model as P

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_ops.npz"))
t = lambda k: torch.from_numpy(G[k])


def test_rms_norm_matches_reference_formula():
    y = P.rms_norm(t("norm_x"), t("norm_w"), float(G["norm_eps"]))
    assert torch.allclose(y, t("norm_y"), atol=1e-6, rtol=1e-6)


def test_rope_matches_reference_formula():
    x = t("rope_x")
    cos, sin = P.rope_cos_sin(t("rope_pos"), x.shape[-1], float(G["rope_theta"]))
    y = P.rope_neox(x, cos.float(), sin.float())
    assert torch.allclose(y, t("rope_y"), atol=1e-6, rtol=1e-6)


def test_attention_matches_reference_formula():
    q, k, v, hist = t("attn_q"), t("attn_k"), t("attn_v"), int(G["attn_hist"])
    qfull = torch.cat([torch.zeros(hist, *q.shape[1:]), q])       # rows before the history do not matter
    o = P.causal_gqa_attention(qfull, k, v, float(G["attn_scale"]))[hist:]
    assert torch.allclose(o, t("attn_o"), atol=1e-5, rtol=1e-5)


def test_window_limits_the_keys():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 2, 8, generator=g, dtype=torch.float64) for _ in range(3))
    full = P.causal_gqa_attention(q, k, v, 0.3)
    w = P.causal_gqa_attention(q, k, v, 0.3, window=4)
    assert torch.allclose(full[:4], w[:4]) and not torch.allclose(full[4:], w[4:])
    last = P.causal_gqa_attention(q[5:], k[5:], v[5:], 0.3)       # row 8 sees keys 5..8 only
    assert torch.allclose(w[8], last[3])


def test_model_is_causal_and_stable_in_32_bit(tmp_path):
    d = H.make_model_dir(str(tmp_path / "m"), H.TINY_B, *H.INIT["B"], torch.float32)
    W = H.load_plain_weights(d)
    ids = [5, 400, 3, 77, 12, 9, 516, 0, 44]
    a = P.qwen3_logits(W, H.TINY_B, ids)
    b = P.qwen3_logits(W, H.TINY_B, ids[:6])
    assert torch.allclose(a[:6], b, atol=1e-12)                   # a prefix's logits ignore what follows
    f32 = P.qwen3_logits(W, H.TINY_B, ids, dtype=torch.float32)
    assert float((f32.double() - a).abs().max() / a.abs().max()) < 1e-5
    assert a.shape == (9, 517)


def test_tied_head_uses_the_embedding(tmp_path):
    d = H.make_model_dir(str(tmp_path / "m"), H.TINY_A, *H.INIT["A"], torch.float32)
    W = H.load_plain_weights(d)
    assert "lm_head.weight" not in W
    a = P.qwen3_logits(W, H.TINY_A, [1, 2, 3])
    W2 = dict(W, **{"lm_head.weight": W["model.embed_tokens.weight"].clone()})
    assert torch.equal(a, P.qwen3_logits(W2, H.TINY_A, [1, 2, 3]))


def test_philox_known_answer():
    # Random123's known-answer vector for philox4x32-10 with zero counter and key: c0 = 0x6627e8d5
    assert P.philox_uniform(0, 0) == (0x6627E8D5 >> 8) / 16777216.0
    us = [P.philox_uniform(7, i) for i in range(2000)]
    assert 0.0 <= min(us) and max(us) < 1.0 and abs(sum(us) / len(us) - 0.5) < 0.03
    assert P.philox_uniform(7, 3) != P.philox_uniform(8, 3)


def test_sampling_rules():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 3.0, 0.0])
    assert P.sample_token(logits, 0.0, 1, 0) == 4
    assert P.sample_token(torch.tensor([1.0, 5.0, 5.0]), 0.0, 1, 0) == 1          # ties to the lowest index
    counts = np.zeros(6)
    for i in range(4000):
        counts[P.sample_token(logits, 0.8, 3, i)] += 1
    want = torch.softmax(logits.double() / 0.8, 0).numpy()
    assert np.abs(counts / 4000 - want).max() < 0.03
    assert {P.sample_token(logits, 1.0, 3, i, top_k=2) for i in range(300)} == {0, 4}
    assert {P.sample_token(logits, 1.0, 3, i, top_p=0.5) for i in range(300)} == {4}
    assert {P.sample_token(logits, 1.0, 3, i, top_p=0.8) for i in range(300)} == {0, 4}
    assert {P.sample_token(logits, 1.0, 3, i, min_p=0.3) for i in range(300)} == {0, 4}
