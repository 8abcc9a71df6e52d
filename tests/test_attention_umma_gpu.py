"""The tcgen05 / TMEM / TMA prompt attention (the kernel with 128-key tiles and the one with 64-key tiles for
short contexts) against the plain formula: portions with and without
history, several requests, both head sizes, group sizes that divide 128, page sizes 8..256, windows,
decoded tokens in the batch left alone, garbage in unused cache slots, a decisive far key."""
import random

import pytest
import torch

from test_kernels_gpu import paged_case, plain_paged

pytestmark = pytest.mark.gpu


def run(reqs, H, Hkv, D, bs, window, seed, key_splits=1, short=False):
    from dinfer_b200.kernels import attention_ops as A
    from dinfer_b200.kernels import gemm_ops as G
    rng = random.Random(seed)
    q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, reqs, H, Hkv, D, bs, torch.bfloat16, window=window)
    seq = torch.tensor([h + n for h, n in reqs], dtype=torch.int32)
    scale = D ** -0.5
    T = q.shape[0]
    wide = torch.zeros(T, (H + 2 * Hkv) * D, dtype=torch.bfloat16, device="cuda")    # q as columns of the qkv rows
    wide[:, :H * D] = q.reshape(T, H * D).cuda()
    out = torch.full((T, H * D), 7.0, dtype=torch.bfloat16, device="cuda")
    bound = A.umma_pair_bound([n for _, n in reqs], H // Hkv) if seed % 2 else 0       # the step's own bound, or none
    if short:
        assert A.umma64_supported(torch.bfloat16, D, H // Hkv, bs)
        A.attention_umma64(wide[:, :H * D], out, cache.cuda(), table.cuda(), cu.cuda(), seq.cuda(), H, Hkv, D, scale,
                           window or 0, max(n for _, n in reqs), bound)
    else:
        A.attention_umma(wide[:, :H * D], out, cache.cuda(), table.cuda(), cu.cuda(), seq.cuda(), H, Hkv, D, scale,
                         window or 0, max(n for _, n in reqs), key_splits, bound)
    G.check_status()
    want = plain_paged(reqs, qs, ks, vs, scale, window).reshape(T, H * D)
    got = out.double().cpu()
    rows = [r for i, (_, n) in enumerate(reqs) if n > 1 for r in range(int(cu[i]), int(cu[i + 1]))]
    skipped = [r for r in range(T) if r not in rows]
    assert torch.isfinite(got).all()
    err = float((got[rows] - want[rows]).abs().max())
    assert err < 2e-2, err
    assert float(torch.nn.functional.cosine_similarity(got[rows], want[rows], dim=-1).min()) > 0.999
    assert bool((got[skipped] == 7.0).all())


@pytest.mark.parametrize("H,Hkv,D,bs", [(8, 2, 128, 16), (4, 4, 128, 8), (16, 1, 128, 64), (8, 4, 64, 16),
                                        (2, 1, 64, 32), (32, 8, 128, 16), (8, 2, 128, 128), (4, 2, 64, 256)])
@pytest.mark.parametrize("window", [None, 70])
def test_mixed_portions(H, Hkv, D, bs, window):
    reqs = [(40, 5), (70, 1), (0, 33), (130, 64), (0, 1), (250, 17), (0, 2), (65, 130), (0, 300)]
    run(reqs, H, Hkv, D, bs, window, seed=H * D + bs)
    if bs <= 64:
        run(reqs, H, Hkv, D, bs, window, seed=H * D + bs + 1, short=True)


@pytest.mark.parametrize("short", [False, True])
def test_long_prompt_and_history(short):
    run([(0, 1100)], 8, 2, 128, 16, None, seed=1, short=short)
    run([(1500, 700), (3, 129)], 8, 2, 128, 16, None, seed=2, short=short)
    run([(900, 260)], 4, 1, 64, 16, 333, seed=3, short=short)


@pytest.mark.parametrize("key_splits", [2, 4, 8])
@pytest.mark.parametrize("H,Hkv,D,bs,window", [(8, 2, 128, 16, None), (4, 4, 128, 8, 300), (8, 4, 64, 16, None),
                                               (2, 1, 64, 32, 70), (16, 1, 128, 64, None)])
def test_keys_split_over_the_ctas_of_a_cluster(H, Hkv, D, bs, window, key_splits):
    """The keys of a row-tile pair dealt out to 2, 4 or 8 CTAs that fold their results through distributed shared
    memory: requests with fewer key tiles than CTAs (some CTAs hold nothing, and for the earliest rows of a prompt
    without history only the first does), a second row tile that does not exist or has a tile less, a window that
    cuts the early tiles away, long histories, decoded tokens left alone."""
    reqs = [(1500, 300), (0, 1), (0, 40), (900, 33), (0, 600), (127, 2), (260, 64), (3000, 1), (640, 129)]
    run(reqs, H, Hkv, D, bs, window, seed=key_splits * 1000 + H * D + bs, key_splits=key_splits)


def test_keys_split_and_a_far_key_in_another_cta():
    """One key decides every row and lies in the first CTA's share; the rows are written by all four CTAs."""
    from dinfer_b200.kernels import attention_ops as A
    from dinfer_b200.kernels import gemm_ops as G
    H, Hkv, D, bs = 4, 2, 128, 16
    rng = random.Random(14)
    hist, new, far = 2000, 128, 37
    q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, [(hist, new)], H, Hkv, D, bs, torch.bfloat16)
    q[:] = 0
    q[:, :, 0] = 100.0
    cache[:, 0, :, :, 0] = 0
    blk = int(table[0, far // bs])
    cache[blk, 0, :, far % bs, 0] = 10.0
    seq = torch.tensor([hist + new], dtype=torch.int32)
    for key_splits in (2, 4, 8):
        out = torch.empty(new, H * D, dtype=torch.bfloat16, device="cuda")
        A.attention_umma(q.reshape(new, H * D).cuda(), out, cache.cuda(), table.cuda(), cu.cuda(), seq.cuda(), H, Hkv, D,
                         1.0, 0, new, key_splits)
        G.check_status()
        want = cache[blk, 1, :, far % bs].float().repeat_interleave(H // Hkv, 0)
        for t in (0, new // 2, new - 1):
            assert torch.allclose(out[t].float().reshape(H, D).cpu(), want, atol=2e-2), (key_splits, t)


def test_many_decoding_requests_beside_a_portion():
    """The grid counts the batch's row-tile pairs, not requests: 300 requests that bring one token each, before,
    between and behind three portions."""
    reqs = [(50 + i, 1) for i in range(120)] + [(700, 200)] + [(9, 1)] * 100 + [(0, 300), (128, 2)] + [(77, 1)] * 80
    run(reqs, 8, 2, 128, 16, None, seed=21, key_splits=2)
    run(reqs, 4, 4, 64, 8, 90, seed=22)
    run(reqs, 8, 2, 128, 16, None, seed=23, short=True)
    run(reqs, 4, 4, 64, 8, 90, seed=24, short=True)


def test_key_split_choice():
    """As many ways as keep every cluster running at once and leave a CTA four key tiles."""
    from dinfer_b200.kernels import attention_ops as A
    assert A.umma_key_splits([1, 1, 1], 4, 8, 128, 4096) == 1              # no portion
    assert A.umma_key_splits([2048], 4, 8, 128, 2048) == 1                 # 256 tile pairs: more than SMs
    assert A.umma_key_splits([64], 4, 8, 128, 256) == 1                    # two tiles: nothing to share
    for lens, seq in (([512, 1, 1], 4096), ([64], 100000), ([256, 300], 8192)):
        got = A.umma_key_splits(lens, 4, 8, 128, seq)
        pairs = sum((n * 4 + 255) // 256 for n in lens if n > 1) * 8
        assert got in (1, 2, 4, 8)
        assert got == 1 or (pairs <= A.umma_max_clusters(128, got) and (seq + 127) // 128 >= got * 4)
        assert got == 8 or (seq + 127) // 128 < got * 8 or pairs > A.umma_max_clusters(128, got * 2)
    assert A.umma_max_clusters(128, 1) >= A.umma_max_clusters(128, 2) * 2 - 2 > 0


@pytest.mark.parametrize("short", [False, True])
def test_more_pages_than_the_shared_memory_table_holds(short):
    """Block tables longer than the slice a CTA keeps in shared memory (2048 entries): the entries
    beyond it are read from the table in memory."""
    run([(17000, 40)], 4, 2, 128, 8, None, seed=5, short=short)
    run([(16500, 300)], 4, 1, 64, 8, 9000, seed=6, short=short)


def test_far_key_wins():
    from dinfer_b200.kernels import attention_ops as A
    H, Hkv, D, bs = 4, 2, 128, 16
    rng = random.Random(4)
    hist, new, far = 700, 50, 37
    q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, [(hist, new)], H, Hkv, D, bs, torch.bfloat16)
    q[:] = 0
    q[:, :, 0] = 100.0
    cache[:, 0, :, :, 0] = 0
    blk = int(table[0, far // bs])
    cache[blk, 0, :, far % bs, 0] = 10.0
    seq = torch.tensor([hist + new], dtype=torch.int32)
    out = torch.empty(new, H * D, dtype=torch.bfloat16, device="cuda")
    A.attention_umma(q.reshape(new, H * D).cuda(), out, cache.cuda(), table.cuda(), cu.cuda(), seq.cuda(), H, Hkv, D,
                     1.0, 0, new)
    want = cache[blk, 1, :, far % bs].float().repeat_interleave(H // Hkv, 0)
    for t in (0, new // 2, new - 1):
        assert torch.allclose(out[t].float().reshape(H, D).cpu(), want, atol=2e-2)


@pytest.mark.parametrize("window", [73, 70, 16, 130])
@pytest.mark.parametrize("H,Hkv,D,bs", [(8, 2, 128, 16), (4, 2, 64, 8), (4, 1, 128, 32), (6, 3, 64, 4)])
def test_window_edges_with_the_passed_pages_given_back(H, Hkv, D, bs, window):
    """Every kernel that walks a block table, with the pages a window has passed given back (-1 in the table, NaN
    wherever no request holds a page): the window's edge on a 64-key tile's edge (history 200, window 73: the
    first key seen is 128), inside a page (window 70), nearer than a page ago (16), and inside a short portion
    whose first rows still see keys the last rows do not."""
    from dinfer_b200.kernels import attention_ops as A
    from dinfer_b200.kernels import gemm_ops as G
    reqs = [(200, 1), (200, 5), (300, 2), (129, 40), (0, 150), (1000, 1), (64, 1), (10, 1)]
    rng = random.Random(window * 1000 + H * D + bs)
    q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, reqs, H, Hkv, D, bs, torch.bfloat16, window=window)
    assert int((table[0] == -1).sum()) > (200 - window) // bs - 1          # pages really are gone
    seq = torch.tensor([h + n for h, n in reqs], dtype=torch.int32)
    scale = D ** -0.5
    T = q.shape[0]
    want = plain_paged(reqs, qs, ks, vs, scale, window).reshape(T, H * D)
    dq, dc, dt, dcu, dseq = q.reshape(T, H * D).cuda(), cache.cuda(), table.cuda(), cu.cuda(), seq.cuda()
    dec = [int(cu[i]) for i, (_, n) in enumerate(reqs) if n == 1]
    pre = [r for i, (_, n) in enumerate(reqs) if n > 1 for r in range(int(cu[i]), int(cu[i + 1]))]
    max_q = max(n for _, n in reqs)

    def held(out, rows, what):
        got = out.double().cpu()[rows]
        assert torch.isfinite(got).all(), what
        assert float((got - want[rows]).abs().max()) < 2e-2, what

    for splits in (1, 4):
        out = torch.full((T, H * D), 7.0, dtype=torch.bfloat16, device="cuda")
        A.attention_decode(dq, out, dc, dt, dcu, dseq, H, Hkv, D, scale, window, splits)      # TMA, or cp.async at pages of 4
        held(out, dec, f"decode kernel, {splits} splits")
        out = torch.full((T, H * D), 7.0, dtype=torch.bfloat16, device="cuda")
        A.attention_tc(dq, out, dc, dt, dcu, dseq, H, Hkv, D, scale, window, max_q, True, True, splits)
        held(out, dec + pre, f"mma.sync kernel, {splits} splits")
    if A.umma_supported(torch.bfloat16, D, H // Hkv, bs):
        out = torch.full((T, H * D), 7.0, dtype=torch.bfloat16, device="cuda")
        A.attention_umma(dq, out, dc, dt, dcu, dseq, H, Hkv, D, scale, window, max_q)
        held(out, pre, "tcgen05 kernel")
        out = torch.full((T, H * D), 7.0, dtype=torch.bfloat16, device="cuda")
        A.attention_umma64(dq, out, dc, dt, dcu, dseq, H, Hkv, D, scale, window, max_q)
        held(out, pre, "tcgen05 kernel with 64-key tiles")
    G.check_status()
