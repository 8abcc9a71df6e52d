"""The decode-attention entry point that allocates nothing (``dinfer_attention_decode_static``).

Some users of this library cannot let it allocate device memory: code that runs inside a CUDA graph
capture, hosts that give the library a fixed budget, plug-ins that must stay away from the host
program's allocator.  For them the split-key decode attention has a twin whose scratch is a fixed
array inside the library.  This test calls that twin through its exported C symbol, twice in a row
(the second call with other inputs and another split count, so that whatever the first call left in
the shared array would show), and holds each result against the regular entry point's.
The file sorts last so that a run that stops at the first failure has already run everything else.
"""
import ctypes
import random
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, reqs, H, Hkv, D, bs):
    from test_kernels_gpu import paged_case
    rng = random.Random(seed)
    q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, reqs, H, Hkv, D, bs, torch.bfloat16)
    seq = torch.tensor([h + n for h, n in reqs], dtype=torch.int32)
    return q.reshape(-1, H * D).cuda(), cache.cuda(), table.cuda(), cu.cuda(), seq.cuda()


def test_static_scratch_entry_point_matches_the_regular_one():
    from dinfer_b200.csrc import build
    from dinfer_b200.kernels import attention_ops as A
    lib = ctypes.CDLL(build.ensure_built(["attention_decode"])["attention_decode"])
    fn = lib.dinfer_attention_decode_static
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    lib.dinfer_last_error.restype = ctypes.c_char_p
    H, Hkv, D, bs = 8, 2, 128, 16
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    for seed, reqs, splits, window in ((1, [(900, 1), (63, 1), (0, 1), (300, 1)], 5, 0),
                                       (2, [(40, 1), (1500, 1), (129, 1)], 3, 200)):
        q, cache, table, cu, seq = _case(seed, reqs, H, Hkv, D, bs)
        B = len(reqs)
        want = torch.zeros(B, H * D, dtype=torch.bfloat16, device="cuda")
        A.attention_decode(q, want, cache, table, cu, seq, H, Hkv, D, D ** -0.5, window, splits)
        got = torch.full((B, H * D), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), cache.data_ptr(), table.data_ptr(),
                table.shape[1], cu.data_ptr(), seq.data_ptr(), B, H, Hkv, D, bs, D ** -0.5, window, splits, stream)
        assert rc == 0, lib.dinfer_last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert float((got.float() - want.float()).abs().max()) < 2e-2
    # beyond the fixed array: refused with a message, nothing launched
    rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), cache.data_ptr(), table.data_ptr(),
            table.shape[1], cu.data_ptr(), seq.data_ptr(), 4096, 64, 8, 128, bs, 0.1, 0, 32, stream)
    assert rc != 0 and b"fixed array" in lib.dinfer_last_error()
