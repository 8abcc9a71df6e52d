"""The tcgen05 / TMA matrix product against a plain f32 product of the same bfloat16 operands: both
orientations, ragged sizes (rows that are no multiple of the tile, K with a tail), K splits, strided
operands, f32 output, and the status word."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def operands(tokens, N, K, seed, pad=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, K + pad, generator=g).to(torch.bfloat16).cuda()[:, :K]
    w = (torch.randn(N, K + pad, generator=g) / math.sqrt(K)).to(torch.bfloat16).cuda()[:, :K]
    return x, w


def check(x, w, out):
    want = x.float() @ w.float().T
    got = out.float()
    assert torch.isfinite(got).all()
    tol = 2e-2 if out.dtype == torch.bfloat16 else 2e-4
    err = float((got - want).abs().max())
    assert err < tol * max(1.0, float(want.abs().max())), (err, float(want.abs().max()))


@pytest.mark.parametrize("tokens", [1, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K", [(128, 64), (256, 256), (517, 96), (1000, 4096), (6144, 1024)])
def test_decode_orientation(tokens, N, K):
    from dinfer_b200.kernels import gemm_ops as G
    x, w = operands(tokens, N, K, tokens * N + K)
    for splits in (1, 2, 3, 5, 7, 8, None):              # the CTAs of a tile share its rows: every cluster size
        out = torch.full((tokens, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        G.gemm_tc(x, w, out, splits=splits)
        check(x, w, out)
    G.check_status()


@pytest.mark.parametrize("tokens,N,K", [(65, 256, 64), (128, 512, 128), (200, 300, 96), (300, 1000, 520),
                                        (2048, 6144, 4096), (1000, 4096, 12288), (4096, 6000, 264), (129, 40000, 72)])
def test_prompt_orientation(tokens, N, K):
    from dinfer_b200.kernels import gemm_ops as G
    x, w = operands(tokens, N, K, tokens + N + K)
    out = torch.full((tokens, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.gemm_tc(x, w, out)
    check(x, w, out)
    G.check_status()


def test_strided_operands_and_f32_output():
    from dinfer_b200.kernels import gemm_ops as G
    x, w = operands(5, 777, 200, 1, pad=24)                # row strides 224 > K
    assert x.stride(0) == 224
    out = torch.empty(5, 777, dtype=torch.float32, device="cuda")
    G.gemm_tc(x, w, out)
    check(x, w, out)
    x, w = operands(100, 333, 200, 2, pad=8)
    wide = torch.zeros(100, 400, dtype=torch.bfloat16, device="cuda")
    G.gemm_tc(x, w, wide[:, 8:341])                          # a column window of a wider output
    check(x, w, wide[:, 8:341])
    assert float(wide[:, :8].abs().max()) == 0 and float(wide[:, 341:].abs().max()) == 0
    outf = torch.empty(100, 333, dtype=torch.float32, device="cuda")
    G.gemm_tc(x, w, outf)
    check(x, w, outf)
    G.check_status()


def test_refuses_what_tma_cannot_address():
    from dinfer_b200.kernels import gemm_ops as G
    from dinfer_b200.kernels.lib import KernelError
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda")      # K = 100 is no multiple of 8
    w = torch.zeros(16, 100, dtype=torch.bfloat16, device="cuda")
    assert not G.supported(x, w)
    with pytest.raises(KernelError):
        G.gemm_tc(x, w, torch.empty(4, 16, dtype=torch.bfloat16, device="cuda"))


def test_repeated_split_launches_agree_bitwise():
    from dinfer_b200.kernels import gemm_ops as G
    x, w = operands(8, 4096, 4096, 9)
    want = x.float() @ w.float().T
    first = None
    for _ in range(5):
        out = torch.empty(8, 4096, dtype=torch.bfloat16, device="cuda")
        G.gemm_tc(x, w, out, splits=8)
        assert float((out.float() - want).abs().max()) < 2e-2 * float(want.abs().max())
        first = out if first is None else first
        assert torch.equal(out, first)                   # the partial sums are added in split order
    G.check_status()


@pytest.mark.parametrize("tokens", [1, 8, 17, 32, 64])
@pytest.mark.parametrize("N,K", [(256, 256), (518, 96), (6144, 1024), (24576, 4096)])
def test_gated_epilogue(tokens, N, K):
    """Weight rows in (gate, up) pairs: out[t, j] = silu(x w_2j) * (x w_2j+1), whatever the K split."""
    from dinfer_b200.kernels import gemm_ops as G
    x, w = operands(tokens, N, K, tokens + N + K)
    y = x.float() @ w.float().T
    want = torch.nn.functional.silu(y[:, 0::2]) * y[:, 1::2]
    for splits in (1, 2, 3, 5, 8, None):
        out = torch.full((tokens, N // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
        G.gemm_tc(x, w, out, splits=splits, gated=True)
        got = out.float()
        assert torch.isfinite(got).all()
        assert float((got - want).abs().max()) < 2e-2 * max(1.0, float(want.abs().max())), splits
    G.check_status()


@pytest.mark.parametrize("tokens,N,K", [(65, 256, 64), (300, 518, 96), (200, 1004, 520), (2048, 24576, 4096),
                                        (1111, 6144, 1024)])
@pytest.mark.parametrize("f32_out", [False, True])
def test_gated_epilogue_of_the_prompt_orientation(tokens, N, K, f32_out):
    """More than 64 rows: persistent pairs of CTAs, each over several tiles; the gate runs in their epilogue."""
    from dinfer_b200.kernels import gemm_ops as G
    x, w = operands(tokens, N, K, tokens + N + K)
    y = x.float() @ w.float().T
    want = torch.nn.functional.silu(y[:, 0::2]) * y[:, 1::2]
    out = torch.full((tokens, N // 2), float("nan"), dtype=torch.float32 if f32_out else torch.bfloat16, device="cuda")
    G.gemm_tc(x, w, out, gated=True)
    got = out.float()
    assert torch.isfinite(got).all()
    tol = (1e-3 if f32_out else 2e-2) * max(1.0, float(want.abs().max()))
    assert float((got - want).abs().max()) < tol
    G.check_status()


@pytest.mark.parametrize("tokens", [1, 8, 17, 33])
@pytest.mark.parametrize("N,K,N2", [(256, 128, 384), (1000, 96, 130), (4096, 4096, 6144), (1024, 3072, 2048)])
def test_norm_taken_apart_between_two_products(tokens, N, K, N2):
    """``residual += x w^T``; the next product's input is the new residual times the norm weight, and its
    result is scaled by 1 / rms of the residual row: together the RMSNorm between the two products."""
    from dinfer_b200.kernels import gemm_ops as G
    g = torch.Generator().manual_seed(tokens + N + K)
    x, w = operands(tokens, N, K, tokens * 3 + N)
    resid = torch.randn(tokens, N, generator=g)
    nw = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.bfloat16).cuda()
    eps = 1e-5
    for splits in (1, 2, 3, None):
        parts = G.residual_parts(tokens, N, K, splits)
        sums = torch.full((parts + 1, 64), float("nan"), device="cuda")
        r = resid.clone().cuda()
        xw = torch.full((tokens, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        G.gemm_tc(x, w, xw, splits=splits, residual=r, norm_weight=nw, sums=sums)
        want_r = resid.cuda() + x.float() @ w.float().T
        assert float((r - want_r).abs().max()) < 1e-3 * max(1.0, float(want_r.abs().max()))
        want_xw = (want_r * nw.float())
        assert float((xw.float() - want_xw).abs().max()) < 1e-2 * max(1.0, float(want_xw.abs().max()))
        ss = sums[:parts, :tokens].sum(0)
        assert torch.allclose(ss, (want_r ** 2).sum(1), rtol=1e-4)
        assert torch.isnan(sums[parts]).all()                   # nothing written beyond the parts
        # the consumer: a plain product and a gated one, scaled by 1 / rms
        w2 = (torch.randn(N2, N, generator=g) / math.sqrt(N)).to(torch.bfloat16).cuda()
        rstd = torch.rsqrt((r ** 2).sum(1) / N + eps)
        y = (xw.float() @ w2.float().T) * rstd[:, None]
        out = torch.full((tokens, N2), float("nan"), dtype=torch.bfloat16, device="cuda")
        G.gemm_tc(xw, w2, out, row_scale=(sums, parts, N, eps))
        assert float((out.float() - y).abs().max()) < 2e-2 * max(1.0, float(y.abs().max()))
        act = torch.full((tokens, N2 // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
        G.gemm_tc(xw, w2, act, gated=True, row_scale=(sums, parts, N, eps))
        want_act = torch.nn.functional.silu(y[:, 0::2]) * y[:, 1::2]
        assert float((act.float() - want_act).abs().max()) < 2e-2 * max(1.0, float(want_act.abs().max()))
    G.check_status()
