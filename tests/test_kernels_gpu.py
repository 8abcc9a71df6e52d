"""Each kernel alone against a plain torch reference of the same operation, at sizes other than the
engine's tiny models (widths and vocabularies that are no power of two, head sizes in steps of 16,
odd head and group counts)."""
import math
import random

import pytest
import torch

import plain_model as P

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]


def tol(dt):
    return dict(atol=2e-5, rtol=2e-5) if dt == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def dev(t, dt=None):
    return t.to("cuda", dtype=dt) if dt else t.to("cuda")


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("T,h", [(1, 24), (7, 1000), (33, 4100), (3, 20000)])
def test_rmsnorm_add_and_gather(dt, T, h):
    from dinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(T * h)
    res = torch.randn(T, h, generator=g) * 3
    delta = (torch.randn(T, h, generator=g)).to(dt)
    w = (1 + 0.3 * torch.randn(h, generator=g)).to(dt)
    eps = 1e-5
    # plain norm of the residual
    r = dev(res.clone())
    out = torch.empty(T, h, dtype=dt, device="cuda")
    ops.rmsnorm(r, dev(w), eps, out)
    want = P.rms_norm(res.double(), w.double(), eps)
    assert torch.allclose(out.double().cpu(), want, **tol(dt))
    assert torch.equal(r.cpu(), res)
    # fused add: residual updated in place, in 32-bit
    ops.rmsnorm(r, dev(w), eps, out, delta=dev(delta))
    summed = res + delta.float()
    assert torch.equal(r.cpu(), summed)
    assert torch.allclose(out.double().cpu(), P.rms_norm(summed.double(), w.double(), eps), **tol(dt))
    # gather of rows (+ pending delta), residual untouched
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32)
    r2 = dev(res.clone())
    out2 = torch.empty(3, h, dtype=dt, device="cuda")
    ops.rmsnorm(r2, dev(w), eps, out2, delta=dev(delta), rows=dev(rows))
    assert torch.equal(r2.cpu(), res)
    assert torch.allclose(out2.double().cpu(), P.rms_norm(summed.double(), w.double(), eps)[rows.long()], **tol(dt))


@pytest.mark.parametrize("dt", DT)
def test_embedding_and_silu(dt):
    from dinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    table = torch.randn(301, 72, generator=g).to(dt)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = torch.empty(5, 72, dtype=torch.float32, device="cuda")
    ops.embedding(dev(ids), dev(table), out)
    assert torch.equal(out.cpu(), table.float()[ids.long()])
    ops.embedding(dev(ids), dev(table), out, scale=8.48528137)    # a model that scales its embedding
    assert torch.allclose(out.cpu(), table.float()[ids.long()] * 8.48528137, rtol=1e-6, atol=0)
    logits = (torch.randn(3, 1001, generator=g) * 40).float()    # a soft cap on logits, in place
    capped = ops.softcap(dev(logits).clone(), 30.0)
    assert torch.allclose(capped.cpu().double(), 30.0 * torch.tanh(logits.double() / 30.0), rtol=1e-5, atol=1e-5)
    x = (torch.randn(9, 2 * 250, generator=g) * 4).to(dt)
    o = torch.empty(9, 250, dtype=dt, device="cuda")
    ops.silu_mul(dev(x), o)
    xd = x.double()
    want = P.silu(xd[:, :250]) * xd[:, 250:]
    assert torch.allclose(o.double().cpu(), want, **tol(dt))
    for inter in (250, 256, 44):                              # gate and up side by side, vector and plain paths
        x = (torch.randn(7, 2 * inter, generator=g) * 4).to(dt)
        o = torch.empty(7, inter, dtype=dt, device="cuda")
        ops.silu_mul(dev(x), o, pairs=True)
        xd = x.double()
        assert torch.allclose(o.double().cpu(), P.silu(xd[:, 0::2]) * xd[:, 1::2], **tol(dt))


@pytest.mark.parametrize("M,N,K", [(1, 37, 50), (8, 130, 999), (9, 260, 70), (130, 129, 1031), (300, 17, 8)])
@pytest.mark.parametrize("adt,wdt,cdt", [(torch.float32,) * 3, (torch.bfloat16, torch.float32, torch.bfloat16),
                                         (torch.float32, torch.bfloat16, torch.float32)])
def test_gemm_f32(M, N, K, adt, wdt, cdt):
    from dinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(M * N + K)
    a = torch.randn(M, K, generator=g).to(adt)
    w = torch.randn(N, K, generator=g).to(wdt)
    out = torch.empty(M, N, dtype=cdt, device="cuda")
    ops.gemm_f32(dev(a), dev(w), out)
    want = a.double() @ w.double().T
    t = dict(atol=1e-4 * math.sqrt(K), rtol=1e-5) if cdt == torch.float32 else dict(atol=5e-2 * math.sqrt(K) / 8, rtol=1e-2)
    assert torch.allclose(out.double().cpu(), want, **t)


def test_gemm_f32_strided_operands():
    from dinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    big = dev(torch.randn(20, 100, generator=g))
    a = big[:, 10:60]                       # row stride 100, 50 columns
    w = dev(torch.randn(31, 50, generator=g))
    outbig = torch.zeros(20, 64, device="cuda")
    ops.gemm_f32(a, w, outbig[:, 3:34])
    assert torch.allclose(outbig[:, 3:34], a @ w.T, atol=1e-4)
    assert float(outbig[:, :3].abs().max()) == 0 and float(outbig[:, 34:].abs().max()) == 0


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("H,Hkv,D,rot,bs", [(4, 1, 16, 16, 4), (6, 2, 32, 32, 16), (5, 5, 48, 48, 8),
                                             (8, 2, 128, 64, 16), (3, 3, 256, 256, 32), (2, 1, 80, 80, 16),
                                             (32, 8, 128, 128, 16), (5, 1, 128, 128, 16), (16, 8, 128, 128, 8),
                                             (6, 2, 64, 64, 16)])
def test_qk_post(dt, H, Hkv, D, rot, bs):
    from dinfer_b200.kernels import ops
    from dinfer_b200.parts.rope import rope_table
    g = torch.Generator().manual_seed(H * D)
    T, nb, eps, theta, maxpos = 11, 9, 1e-5, 12345.0, 300
    width = (H + 2 * Hkv) * D
    qkv = torch.randn(T, width + 8, generator=g).to(dt)           # padded rows: stride != width
    pos = torch.tensor(random.Random(1).sample(range(maxpos), T), dtype=torch.int32)
    wq = (1 + 0.2 * torch.randn(D, generator=g)).to(dt)
    wk = (1 + 0.2 * torch.randn(D, generator=g)).to(dt)
    slots = torch.tensor(random.Random(2).sample(range(nb * bs), T), dtype=torch.int32)
    slots[3] = -1
    cache = torch.zeros(nb, 2, Hkv, bs, D, dtype=dt, device="cuda")
    table = rope_table(rot, theta, maxpos, "cuda")
    x = dev(qkv)
    ops.qk_post(x[:, :width], dev(pos), H, Hkv, D, eps, dev(wq), dev(wk), table, cache, dev(slots), bs)
    # plain
    q = qkv[:, :H * D].double().reshape(T, H, D)
    k = qkv[:, H * D:(H + Hkv) * D].double().reshape(T, Hkv, D)
    v = qkv[:, (H + Hkv) * D:width].double().reshape(T, Hkv, D)
    cos, sin = P.rope_cos_sin(pos, rot, theta)
    qn, kn = P.rms_norm(q, wq.double(), eps), P.rms_norm(k, wk.double(), eps)
    qn = torch.cat([P.rope_neox(qn[..., :rot], cos, sin), qn[..., rot:]], -1)
    kn = torch.cat([P.rope_neox(kn[..., :rot], cos, sin), kn[..., rot:]], -1)
    got = x.double().cpu()
    assert torch.allclose(got[:, :H * D].reshape(T, H, D), qn, **tol(dt))
    assert torch.allclose(got[:, H * D:(H + Hkv) * D].reshape(T, Hkv, D), kn, **tol(dt))
    assert torch.equal(got[:, (H + Hkv) * D:], qkv[:, (H + Hkv) * D:].double())      # v and the padding untouched
    c = cache.double().cpu()
    want_c = torch.zeros_like(c)
    for t in range(T):
        s = int(slots[t])
        if s >= 0:
            want_c[s // bs, 0, :, s % bs] = kn[t]
            want_c[s // bs, 1, :, s % bs] = v[t]
    assert torch.allclose(c, want_c, **tol(dt))


def paged_case(rng, reqs, H, Hkv, D, bs, dt, extra_blocks=3, window=None):
    """reqs = [(history, new)].  Returns the kernel's inputs and the plain answer [T, H, D].

    With ``window`` the pages that the window has passed before this step are gone, as the cache manager leaves
    them: a page wholly below ``history - window + 1`` has the table entry -1 and its keys are nowhere; every page
    no request holds (page 0 among them, where a kernel that mistook -1 for a page id might look) is NaN, so a
    kernel that reads a key it must not see shows."""
    g = torch.Generator().manual_seed(rng.randrange(1 << 30))
    total_blocks = sum((h + n + bs - 1) // bs for h, n in reqs) + extra_blocks
    perm = list(range(1 if window else 0, total_blocks))
    rng.shuffle(perm)
    cache = (torch.randn(total_blocks, 2, Hkv, bs, D, generator=g) * 50).to(dt)   # garbage where nothing is stored
    if window:
        cache[:] = float("nan")
    max_blocks = max((h + n + bs - 1) // bs for h, n in reqs) + 1
    table = torch.full((len(reqs), max_blocks), -1, dtype=torch.int32)
    qs, ks, vs, pos, cu = [], [], [], [], [0]
    for b, (hist, new) in enumerate(reqs):
        L = hist + new
        k = torch.randn(L, Hkv, D, generator=g).to(dt)
        v = torch.randn(L, Hkv, D, generator=g).to(dt)
        q = torch.randn(new, H, D, generator=g).to(dt)
        first = max(0, hist - window + 1) // bs if window else 0      # pages before it were given back
        for i in range(first, (L + bs - 1) // bs):
            blk = perm.pop()
            table[b, i] = blk
            n = min(bs, L - i * bs)
            cache[blk] = (torch.randn(2, Hkv, bs, D, generator=g) * 50).to(dt)    # what an earlier holder left
            cache[blk, 0, :, :n] = k[i * bs:i * bs + n].transpose(0, 1)
            cache[blk, 1, :, :n] = v[i * bs:i * bs + n].transpose(0, 1)
        qs.append(q); ks.append(k); vs.append(v)
        pos += list(range(hist, L))
        cu.append(cu[-1] + new)
    return (torch.cat(qs), cache, table, torch.tensor(cu, dtype=torch.int32), torch.tensor(pos, dtype=torch.int32),
            qs, ks, vs)


def plain_paged(reqs, qs, ks, vs, scale, window=None):
    outs = []
    for (hist, new), q, k, v in zip(reqs, qs, ks, vs):
        qfull = torch.cat([torch.zeros(hist, *q.shape[1:], dtype=torch.float64), q.double()])
        outs.append(P.causal_gqa_attention(qfull, k.double(), v.double(), scale, window)[hist:])
    return torch.cat(outs)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("H,Hkv,D,bs,window", [(4, 1, 16, 4, None), (6, 2, 32, 16, None), (5, 5, 48, 8, 7),
                                                (8, 2, 128, 16, None), (3, 1, 80, 16, 33), (2, 2, 256, 32, None)])
def test_attention_generic(dt, H, Hkv, D, bs, window):
    from dinfer_b200.kernels import ops
    rng = random.Random(H * 1000 + D)
    reqs = [(40, 5), (70, 1), (0, 33), (130, 64), (0, 1), (7, 1)]        # portions with history beside decodes
    q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, reqs, H, Hkv, D, bs, dt, window=window)
    scale = D ** -0.5
    out = torch.empty(q.shape[0], H * D, dtype=dt, device="cuda")
    ops.attention_generic(dev(q).reshape(-1, H * D), out, dev(cache), dev(table), dev(cu), dev(pos), H, Hkv, D,
                          scale, window or 0)
    want = plain_paged(reqs, qs, ks, vs, scale, window).reshape(-1, H * D)
    assert torch.allclose(out.double().cpu(), want, **tol(dt))


def test_attention_finds_a_far_key():
    """One key among hundreds, on another page, is made to dominate: the output must be its value."""
    from dinfer_b200.kernels import ops
    rng = random.Random(9)
    H, Hkv, D, bs = 4, 2, 64, 16
    reqs = [(600, 1), (300, 2)]
    q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, reqs, H, Hkv, D, bs, torch.float32)
    far = 37                                                  # position of the key that must win, request 0
    q[0] = 0
    q[0, :, 0] = 100.0
    blk = int(table[0, far // bs])
    cache[:, 0, :, :, 0] = 0                                  # no other key has weight along dim 0
    cache[blk, 0, :, far % bs, 0] = 10.0
    out = torch.empty(q.shape[0], H * D, device="cuda")
    ops.attention_generic(dev(q).reshape(-1, H * D), out, dev(cache), dev(table), dev(cu), dev(pos), H, Hkv, D, 1.0, 0)
    got = out[0].reshape(H, D).cpu()
    want = cache[blk, 1, :, far % bs].repeat_interleave(H // Hkv, 0)
    assert torch.allclose(got, want, atol=1e-5)


@pytest.mark.parametrize("V", [517, 4099, 151936])
def test_argmax_and_sampling(V):
    from dinfer_b200.sampling import sampler as S
    g = torch.Generator().manual_seed(V)
    R = 6
    logits = torch.randn(R, V, generator=g) * 3
    logits[2, 11] = logits[2, 400] = 50.0                     # a tie: the lower index wins
    d = dev(logits)
    assert S.argmax(d).cpu().tolist() == [int(torch.argmax(logits[i])) if i != 2 else 11 for i in range(R)]
    temps = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.8, 1.0])
    topk = torch.tensor([-1, -1, 5, -1, 40, 3], dtype=torch.int32)
    topp = torch.tensor([1.0, 1.0, 1.0, 0.6, 0.9, 0.5])
    minp = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.02, 0.0])
    agree = total = 0
    for off in range(25):
        seeds = torch.tensor([7, 8, 9, 10, 11, 12], dtype=torch.int64)
        offs = torch.full((R,), off, dtype=torch.int64)
        got = S.sample(d, dev(temps), dev(seeds), dev(offs), top_k=dev(topk), top_p=dev(topp), min_p=dev(minp)).cpu()
        for i in range(R):
            want = P.sample_token(logits[i], float(temps[i]), int(seeds[i]), off, int(topk[i]), float(topp[i]),
                                  float(minp[i]))
            total += 1
            agree += int(got[i]) == want
    # f32 sums against f64: a draw that lands within rounding of a boundary may pick the neighbour
    assert agree >= total - 2, f"{agree}/{total}"


@pytest.mark.parametrize("R,V,ld", [(64, 151936, 151936), (41, 517, 517), (100, 4099, 4104), (40, 1000, 1001)])
def test_argmax_of_many_rows(R, V, ld):
    """From 40 rows on the argmax runs a CTA per row: every row, ties to the lowest index, rows that start on no
    16-byte boundary, a vocabulary that is no multiple of four, columns beyond the vocabulary ignored."""
    from dinfer_b200.sampling import sampler as S
    g = torch.Generator().manual_seed(R + V)
    full = torch.randn(R, ld, generator=g) * 3
    full[:, V:] = 1e9                                         # beyond the vocabulary: must not be looked at
    logits = full[:, :V]
    logits[3, 5] = logits[3, V - 1] = 60.0                    # a tie: the lower index wins
    logits[7, V - 1] = 70.0                                   # the last column
    logits[8, 0] = 70.0
    got = S.argmax(dev(full)[:, :V]).cpu().tolist()
    want = [int(torch.argmax(logits[i])) for i in range(R)]
    want[3] = 5
    assert got == want


def test_sampling_distribution_and_batch_independence():
    from dinfer_b200.sampling import sampler as S
    logits = torch.tensor([[2.0, 1.0, 0.5, -1.0, 3.0, 0.0, -30.0]])
    n = 3000
    d = dev(logits.repeat(n, 1))
    temps = dev(torch.full((n,), 0.8))
    seeds = dev(torch.full((n,), 123, dtype=torch.int64))
    offs = dev(torch.arange(n, dtype=torch.int64))
    got = S.sample(d, temps, seeds, offs).cpu()
    freq = torch.bincount(got.long(), minlength=7).double() / n
    want = torch.softmax(logits[0].double() / 0.8, 0)
    assert float((freq - want).abs().max()) < 0.03
    # the same (seed, offset) gives the same token wherever the row stands in the batch
    perm = torch.randperm(n)
    got2 = S.sample(d, temps, seeds, dev(torch.arange(n, dtype=torch.int64)[perm])).cpu()
    assert torch.equal(got2, got[perm])


def test_penalties():
    from dinfer_b200.sampling import sampler as S
    V = 50
    logits = torch.linspace(-2, 2, V).repeat(2, 1)
    ids = torch.tensor([3, 40, 40, 7, 40, 3,   1, 2], dtype=torch.int32)     # row 0: prompt [3, 40], output [40, 7, 40, 3]
    offsets = torch.tensor([0, 6, 8], dtype=torch.int32)
    plen = torch.tensor([2, 2], dtype=torch.int32)
    rep, freq, pres = torch.tensor([1.5, 1.0]), torch.tensor([0.3, 0.0]), torch.tensor([0.2, 0.0])
    d = dev(logits.clone())
    S.apply_penalties(d, dev(ids), dev(offsets), dev(plen), dev(rep), dev(freq), dev(pres))
    want = torch.stack([P.penalties(logits[0], [3, 40], [40, 7, 40, 3], 1.5, 0.3, 0.2),
                        P.penalties(logits[1], [1, 2], [], 1.0, 0.0, 0.0)])
    assert not torch.equal(want[0], logits[0]) and torch.equal(want[1], logits[1])
    assert torch.allclose(d.cpu(), want, atol=1e-6)


@pytest.mark.parametrize("V,ld", [(517, 517), (151936, 151936), (1000, 1024)])
@pytest.mark.parametrize("k", [0, 5, 32])
def test_logprobs_and_logit_bias(V, ld, k):
    """Log-probabilities of the chosen token, its rank and the k most likely tokens against log_softmax / topk;
    ties go to the lower id; additive biases land on the given (row, token) pairs only."""
    from dinfer_b200.sampling import sampler as S
    g = torch.Generator().manual_seed(V + k)
    R = 5
    full = (torch.randn(R, ld, generator=g) * 4).cuda()
    logits = full[:, :V]
    logits[1, 7] = logits[1, 3] = float(logits[1].max()) + 1.0          # a tie at the top: id 3 comes first
    logits[2, V - 1] = float("-inf")
    chosen = torch.tensor([0, 7, V - 2, 11, V // 2], dtype=torch.int32, device="cuda")
    ids, lp, rank = S.logprobs(logits, chosen, k)
    want = torch.log_softmax(logits.double(), dim=-1)
    for r in range(R):
        c = int(chosen[r])
        assert int(ids[r, 0]) == c and abs(float(lp[r, 0]) - float(want[r, c])) < 1e-4
        assert int(rank[r]) == int((logits[r] > logits[r, c]).sum())
        if k:
            order = sorted(range(V), key=lambda i: (-float(logits[r, i]), i))[:k]
            assert ids[r, 1:].tolist() == order
            assert torch.allclose(lp[r, 1:].double().cpu(), want[r, order].cpu(), atol=1e-4)
    assert ids[1, 1:3].tolist() == [3, 7][:k] if k else True
    before = logits.clone()
    rows = torch.tensor([0, 0, 3, 4], dtype=torch.int32, device="cuda")
    toks = torch.tensor([1, V - 1, 5, 0], dtype=torch.int32, device="cuda")
    bias = torch.tensor([2.5, -100.0, 100.0, 0.25], device="cuda")
    S.logit_bias(logits, rows, toks, bias)
    want_b = before.clone()
    for r_, t_, b_ in zip(rows.tolist(), toks.tolist(), bias.tolist()):
        want_b[r_, t_] += b_
    assert torch.equal(logits, want_b)
    assert torch.equal(full[:, V:], full[:, V:])                        # the padding of the rows is untouched


def test_top_k_the_short_way_and_its_fallbacks():
    """A small k takes the candidate list, a large one or a crowded bin the radix descent; fewer kept entries than
    k keep them all.  Every way must keep the same set as the plain sampler: same tokens for the same draws."""
    from dinfer_b200.sampling import sampler as S
    g = torch.Generator().manual_seed(77)
    V = 20011
    rows = []
    base = torch.randn(V, generator=g) * 3
    rows.append((base.clone(), 512, 1.0, 0.0))                 # the largest k of the short way
    rows.append((base.clone(), 513, 0.9, 0.0))                 # just beyond it: radix
    crowded = base.clone()
    crowded[100:6100] = float(base.max()) + 1.0                # 6000 equal values at the top: the bin overflows
    rows.append((crowded, 10, 1.0, 0.0))                       # (all 6000 ties are kept)
    rows.append((base.clone(), 50, 0.7, 0.3))                  # min_p leaves fewer than k
    tied = base.clone()
    tied[[5, 900, 15000]] = float(base.max()) + 2.0            # ties across the k-th place are all kept
    rows.append((tied, 2, 1.0, 0.0))
    rows.append((base.clone(), 1, 0.5, 0.0))
    logits = torch.stack([r[0] for r in rows])
    R = len(rows)
    d = dev(logits)
    temps = torch.full((R,), 0.9)
    topk = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    topp = torch.tensor([r[2] for r in rows])
    minp = torch.tensor([r[3] for r in rows])
    agree = total = 0
    for off in range(30):
        seeds = torch.arange(R, dtype=torch.int64) + 3
        offs = torch.full((R,), off, dtype=torch.int64)
        got = S.sample(d, dev(temps), dev(seeds), dev(offs), top_k=dev(topk), top_p=dev(topp), min_p=dev(minp)).cpu()
        for i in range(R):
            want = P.sample_token(logits[i], float(temps[i]), int(seeds[i]), off, int(topk[i]), float(topp[i]),
                                  float(minp[i]))
            total += 1
            agree += int(got[i]) == want
    assert agree >= total - 2, f"{agree}/{total}"
    got = S.sample(d, dev(temps), dev(seeds), dev(offs), top_k=dev(topk), top_p=dev(topp), min_p=dev(minp)).cpu()
    assert int(got[5]) == int(torch.argmax(base)) and int(got[4]) in (5, 900, 15000)
    # top-p over thousands of exact ties: the threshold keeps all entries of a value or none (as the reference's
    # kernel does, crates/kernels/cuda/sampling.cu:99-124), where a sort would cut through them
    topp2 = topp.clone()
    topp2[2] = 0.8
    seen = set()
    for off in range(40):
        offs = torch.full((R,), off, dtype=torch.int64)
        seen.add(int(S.sample(d, dev(temps), dev(seeds), dev(offs), top_k=dev(topk), top_p=dev(topp2), min_p=dev(minp)).cpu()[2]))
    assert all(100 <= t < 6100 for t in seen) and max(seen) > 100 + 0.9 * 6000


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_attention_generic_without_pages(dt):
    """A request whose table holds no page (a dummy row of a captured graph) has no keys: its output is zero and
    nothing outside the cache is read; the request beside it is untouched by it."""
    from dinfer_b200.kernels import ops
    H_, Hkv, D, bs = 4, 2, 24, 4
    g = torch.Generator().manual_seed(5)
    cache = dev(torch.randn(6, 2, Hkv, bs, D, generator=g)).to(dt)
    q = dev(torch.randn(2, H_ * D, generator=g)).to(dt)
    out = torch.full((2, H_ * D), float("nan"), dtype=dt, device="cuda")
    table = dev(torch.tensor([[-1, -1], [3, 1]], dtype=torch.int32))
    cu = dev(torch.tensor([0, 1, 2], dtype=torch.int32))
    pos = dev(torch.tensor([0, 5], dtype=torch.int32))
    ops.attention_generic(q, out, cache, table, cu, pos, H_, Hkv, D, D ** -0.5, 0)
    assert torch.equal(out[0].float(), torch.zeros(H_ * D, device="cuda"))
    alone = torch.empty((1, H_ * D), dtype=dt, device="cuda")
    ops.attention_generic(q[1:], alone, cache, table[1:], dev(torch.tensor([0, 1], dtype=torch.int32)), pos[1:],
                          H_, Hkv, D, D ** -0.5, 0)
    assert torch.equal(out[1], alone[0]) and torch.isfinite(out[1].float()).all()
