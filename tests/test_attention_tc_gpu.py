"""The tensor-core attention kernels against the plain formula: prompt portions with history beside
decoded tokens, every supported head size, odd group sizes, windows, key splits, scattered pages
with garbage in the unused slots."""
import random

import pytest
import torch

from test_kernels_gpu import paged_case, plain_paged

pytestmark = pytest.mark.gpu


def run_tc(reqs, H, Hkv, D, bs, window, splits, seed):
    from dinfer_b200.kernels import attention_ops as A
    rng = random.Random(seed)
    q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, reqs, H, Hkv, D, bs, torch.bfloat16, window=window)
    seq = torch.tensor([h + n for h, n in reqs], dtype=torch.int32)
    scale = D ** -0.5
    # q as columns of a wider row, the way the engine passes the q part of the qkv rows
    wide = torch.zeros(q.shape[0], H * D + 2 * Hkv * D, dtype=torch.bfloat16, device="cuda")
    wide[:, :H * D] = q.reshape(-1, H * D).cuda()
    out = torch.full((q.shape[0], H * D), float("nan"), dtype=torch.bfloat16, device="cuda")
    lens = [n for _, n in reqs]
    A.attention_tc(wide[:, :H * D], out, cache.cuda(), table.cuda(), cu.cuda(), seq.cuda(), H, Hkv, D, scale,
                   window or 0, max(lens), any(n == 1 for n in lens), any(n > 1 for n in lens), splits)
    want = plain_paged(reqs, qs, ks, vs, scale, window).reshape(-1, H * D)
    got = out.double().cpu()
    assert torch.isfinite(got).all()
    err = float((got - want).abs().max())
    assert err < 2e-2, err
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert float(cos.min()) > 0.999


MIXED = [(40, 5), (70, 1), (0, 33), (130, 64), (0, 1), (7, 1), (250, 17), (0, 2), (63, 1), (64, 1), (65, 130)]


@pytest.mark.parametrize("H,Hkv,D,bs", [(6, 2, 32, 16), (4, 4, 64, 4), (8, 1, 64, 16), (8, 2, 128, 16),
                                        (5, 5, 128, 8), (16, 1, 128, 32), (12, 4, 32, 1)])
@pytest.mark.parametrize("window", [None, 37])
def test_mixed_batch(H, Hkv, D, bs, window):
    run_tc(MIXED, H, Hkv, D, bs, window, splits=3, seed=H * D + bs)


@pytest.mark.parametrize("splits", [1, 2, 5, 32])
def test_decode_splits(splits):
    reqs = [(1000, 1), (63, 1), (0, 1), (129, 1), (4095, 1)]
    run_tc(reqs, 8, 2, 128, 16, None, splits, seed=splits)
    run_tc(reqs, 8, 2, 128, 16, 100, splits, seed=splits + 100)


@pytest.mark.parametrize("H,Hkv,D,bs", [(8, 2, 128, 16), (32, 8, 128, 16), (3, 3, 128, 4), (8, 1, 64, 32),
                                        (16, 1, 128, 16), (12, 1, 64, 1), (10, 2, 64, 8)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("splits", [1, 2, 3, 4, 5, 6, 7, 9, 12, 16])     # every cluster size the engine can pick
def test_decode_kernel(H, Hkv, D, bs, window, splits):
    """The decode kernel (keys on the tile's rows, splits folded in the kernel) against the plain
    formula; a prompt portion in the batch must be left alone; two launches in a row (the splits fold
    through a cluster's shared memory, or through a scratch that every launch leaves clean)."""
    from dinfer_b200.kernels import attention_ops as A
    from test_kernels_gpu import paged_case, plain_paged
    reqs = [(1000, 1), (63, 1), (0, 1), (129, 1), (40, 6), (2047, 1), (64, 1), (15, 1)]
    rng = random.Random(H * D + bs + splits)
    q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, reqs, H, Hkv, D, bs, torch.bfloat16, window=window)
    seq = torch.tensor([h + n for h, n in reqs], dtype=torch.int32)
    scale = D ** -0.5
    want = plain_paged(reqs, qs, ks, vs, scale, window).reshape(-1, H * D)
    dec_rows = [int(cu[i]) for i, (_, n) in enumerate(reqs) if n == 1]
    other = [r for r in range(q.shape[0]) if r not in dec_rows]
    dq, dc, dt, dcu, dseq = q.reshape(-1, H * D).cuda(), cache.cuda(), table.cuda(), cu.cuda(), seq.cuda()
    for _ in range(2):
        out = torch.full((q.shape[0], H * D), 7.0, dtype=torch.bfloat16, device="cuda")
        A.attention_decode(dq, out, dc, dt, dcu, dseq, H, Hkv, D, scale, window or 0, splits)
        got = out.double().cpu()
        assert torch.isfinite(got).all()
        assert float((got[dec_rows] - want[dec_rows]).abs().max()) < 2e-2
        assert float(torch.nn.functional.cosine_similarity(got[dec_rows], want[dec_rows], dim=-1).min()) > 0.999
        assert bool((got[other] == 7.0).all())


def test_long_prompt_portions():
    run_tc([(0, 700), (900, 300)], 8, 2, 128, 16, None, 1, seed=1)
    run_tc([(0, 700), (900, 300)], 3, 1, 64, 16, 257, 1, seed=2)


def test_far_key_and_window_edge():
    """Scores made decisive: one far key must win; with a window it must be invisible exactly when it
    is ``window`` or more positions back."""
    from dinfer_b200.kernels import attention_ops as A
    H, Hkv, D, bs = 4, 2, 64, 16
    rng = random.Random(4)
    for hist, new, far, window in ((600, 1, 37, None), (300, 40, 5, None), (600, 1, 590, 11), (600, 1, 590, 10)):
        reqs = [(hist, new)]
        q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, reqs, H, Hkv, D, bs, torch.bfloat16, window=window)
        q[:] = 0
        q[:, :, 0] = 100.0
        cache[:, 0, :, :, 0] = 0
        blk = int(table[0, far // bs])
        cache[blk, 0, :, far % bs, 0] = 10.0
        seq = torch.tensor([hist + new], dtype=torch.int32)
        out = torch.empty(new, H * D, dtype=torch.bfloat16, device="cuda")
        A.attention_tc(q.reshape(new, H * D).cuda(), out, cache.cuda(), table.cuda(), cu.cuda(), seq.cuda(), H, Hkv, D,
                       1.0, window or 0, new, new == 1, new > 1, 4)
        got = out[-1].float().reshape(H, D).cpu()
        far_value = cache[blk, 1, :, far % bs].float().repeat_interleave(H // Hkv, 0)
        visible = window is None or far > hist + new - 1 - window
        if visible:
            assert torch.allclose(got, far_value, atol=2e-2), (hist, new, far, window)
        else:
            assert not torch.allclose(got, far_value, atol=0.2), (hist, new, far, window)


def test_decode_kernel_with_more_pages_than_its_shared_memory_table():
    """A context of more than 2048 pages: the page ids beyond the slice in shared memory come from the
    table in memory (one split, and as many as the largest cluster)."""
    from dinfer_b200.kernels import attention_ops as A
    from dinfer_b200.kernels import gemm_ops as G
    from test_kernels_gpu import paged_case, plain_paged
    H, Hkv, D, bs = 8, 2, 128, 8
    reqs = [(17500, 1), (30, 1)]
    rng = random.Random(77)
    q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, reqs, H, Hkv, D, bs, torch.bfloat16)
    seq = torch.tensor([h + n for h, n in reqs], dtype=torch.int32)
    want = plain_paged(reqs, qs, ks, vs, D ** -0.5, None).reshape(-1, H * D)
    for splits in (1, 16):
        out = torch.zeros(q.shape[0], H * D, dtype=torch.bfloat16, device="cuda")
        A.attention_decode(q.reshape(-1, H * D).cuda(), out, cache.cuda(), table.cuda(), cu.cuda(), seq.cuda(),
                           H, Hkv, D, D ** -0.5, 0, splits)
        G.check_status()
        assert float((out.double().cpu() - want).abs().max()) < 2e-2
