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


def bf(x):
    return x.to(torch.bfloat16).float()


def rounds_to(plain: torch.Tensor, want: torch.Tensor) -> bool:
    """``want`` is a bfloat16 value of the reference; the plain result must round to it (a last place apart where
    the unrounded values straddle a rounding boundary, in one entry in a hundred at most)."""
    got = bf(plain.float())
    exact = float((got == want).float().mean())
    return exact >= 0.99 and torch.allclose(got, want, rtol=2.0 ** -7, atol=1e-6)


def test_residual_add_and_norm_match_what_the_references_check_expects():
    res, normed = P.add_and_norm(t("addnorm_res").double(), t("addnorm_x").double(), t("addnorm_w").double(), 1e-5)
    assert rounds_to(res, t("addnorm_res_out"))
    # the reference norms the ROUNDED sum (it keeps the residual in bfloat16); the plain sum is not rounded
    assert torch.allclose(normed.float(), t("addnorm_out"), rtol=2.0 ** -6, atol=2e-3)
    _, normed_r = P.add_and_norm(t("addnorm_res_out").double(), torch.zeros(1, dtype=torch.float64),
                                 t("addnorm_w").double(), 1e-5)
    assert rounds_to(normed_r, t("addnorm_out"))


def test_gate_comes_first():
    x = t("gate_x")
    assert rounds_to(P.gate(x.double()), t("gate_out"))
    i = x.shape[1] // 2
    swapped = P.gate(torch.cat([x[:, i:], x[:, :i]], 1).double())
    assert not torch.allclose(bf(swapped.float()), t("gate_out"), atol=1e-2)


def test_head_norm_comes_before_the_rotation_and_the_cache_gets_rotated_keys():
    H, HK, D = (int(v) for v in G["qkpost_dims"])
    qkv, pos, theta = t("qkpost_qkv"), t("qkpost_pos"), float(G["qkpost_theta"])
    rows, kv = P.qk_post(qkv.double(), pos, H, HK, D, t("qkpost_wq").double(), t("qkpost_wk").double(), 1e-5, theta)
    assert rounds_to(rows, t("qkpost_rows"))
    want_cache = t("qkpost_cache")                            # [slot, kv head, k|v, D], zero where nothing is written
    cache = torch.zeros_like(want_cache)
    for i, sl in enumerate(G["qkpost_slots"].tolist()):
        if sl >= 0:
            cache[sl] = bf(kv[i].float())
    assert rounds_to(cache, want_cache)
    assert float(want_cache.abs().sum(dim=(1, 2, 3)).gt(0).sum()) == 8          # the token without a slot wrote nothing
    # the other order (rotation first) is not what the reference expects
    T = qkv.shape[0]
    cos, sin = P.rope_cos_sin(pos, D, theta)
    q = qkv[:, :H * D].reshape(T, H, D).double()
    wrong = P.rms_norm(P.rope_neox(q, cos, sin), t("qkpost_wq").double(), 1e-5).reshape(T, -1)
    assert not torch.allclose(bf(wrong.float()), t("qkpost_rows")[:, :H * D], atol=5e-2)


def test_penalties_match_the_reference_formula():
    logits, ids = t("pen_logits"), G["pen_ids"].tolist()
    offs, plen = G["pen_offsets"].tolist(), G["pen_prompt_len"].tolist()
    for b in range(logits.shape[0]):
        row = ids[offs[b]:offs[b + 1]]
        got = P.penalties(logits[b], row[:plen[b]], row[plen[b]:], float(G["pen_rep"][b]), float(G["pen_freq"][b]),
                          float(G["pen_pres"][b]))
        assert torch.allclose(got, t("pen_out")[b], atol=1e-6)
    assert not torch.equal(t("pen_out"), logits)


def test_top_k_and_top_p_filters_match_the_reference_formula():
    row = t("filter_row")
    for (kk, pp), want in zip(G["filter_cases"].tolist(), t("filter_out")):
        got = P.filter_logits(row.double(), top_k=int(kk) if kk else -1, top_p=float(pp))
        assert torch.equal(torch.isinf(got), torch.isinf(want)), (kk, pp)
        kept = ~torch.isinf(want)
        assert torch.allclose(got[kept].float(), want[kept])


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
