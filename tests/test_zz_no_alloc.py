"""The decode-attention entry point that allocates nothing (``dinfer_attention_decode_static``).

Some users of this library cannot let it allocate device memory: hosts that give the library a fixed budget,
plug-ins that must stay away from the host program's allocator, loops that cannot afford the device-wide
synchronisation an allocation may bring.  For them the split-key decode attention has a twin whose scratch is a
fixed array inside the library.  This test calls that twin through its exported C symbol, several times in a row
(every call with other inputs, sizes and split counts, so that whatever the last call left in the shared array
would show), and holds each result against the plain attention formula and against the regular entry point given
scratch by the caller (the same kernel, so the two must agree to the bit).
The file sorts last so that a run that stops at the first failure has already run everything else.
"""
import ctypes
import random
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_against_the_plain_formula_and_the_regular_one():
    from dinfer_b200.csrc import build
    from test_kernels_gpu import paged_case, plain_paged
    lib = ctypes.CDLL(build.ensure_built(["attention_decode"])["attention_decode"])
    fn = lib.dinfer_attention_decode_static
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    regular = lib.dinfer_attention_decode
    regular.restype = c_int
    regular.argtypes = fn.argtypes[:-1] + [c_void_p, c_void_p, c_void_p]
    lib.dinfer_last_error.restype = ctypes.c_char_p
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    cases = [  # seed, (H, Hkv, D, page), requests (history, 1), splits, window
        (1, (8, 2, 128, 16), [(900, 1), (63, 1), (0, 1), (300, 1)], 5, 0),
        (2, (8, 2, 128, 16), [(40, 1), (1500, 1), (129, 1)], 3, 200),
        (3, (8, 2, 128, 16), [(700, 1), (5, 1)], 1, 0),                    # one split: no scratch, no clearing
        (4, (12, 1, 64, 4), [(333, 1), (64, 1), (1000, 1)], 4, 0),         # head size 64, a group of 12, pages of 4
        (5, (12, 1, 64, 4), [(20, 1), (260, 1)], 7, 90),
    ]
    for seed, (H, Hkv, D, bs), reqs, splits, window in cases:
        rng = random.Random(seed)
        q, cache, table, cu, pos, qs, ks, vs = paged_case(rng, reqs, H, Hkv, D, bs, torch.bfloat16,
                                                          window=window or None)
        want = plain_paged(reqs, qs, ks, vs, D ** -0.5, window or None).reshape(-1, H * D)
        B = len(reqs)
        q, cache, table, cu = q.reshape(-1, H * D).cuda(), cache.cuda(), table.cuda(), cu.cuda()
        seq = torch.tensor([h + n for h, n in reqs], dtype=torch.int32, device="cuda")
        got = torch.full((B, H * D), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), cache.data_ptr(), table.data_ptr(),
                table.shape[1], cu.data_ptr(), seq.data_ptr(), B, H, Hkv, D, bs, D ** -0.5, window, splits, stream)
        assert rc == 0, lib.dinfer_last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all(), (seed, "not finite")
        err = float((got.double().cpu() - want).abs().max())
        assert err < 2e-2, (seed, err)                                      # the tolerance of the kernel tests
        # the regular entry point with the caller's scratch: the same kernel, the same bits
        floats = torch.empty(B * H * splits * (D + 2), dtype=torch.float32, device="cuda")
        counters = torch.zeros(B * Hkv, dtype=torch.int32, device="cuda")
        ref = torch.full((B, H * D), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = regular(q.data_ptr(), q.stride(0), ref.data_ptr(), ref.stride(0), cache.data_ptr(), table.data_ptr(),
                     table.shape[1], cu.data_ptr(), seq.data_ptr(), B, H, Hkv, D, bs, D ** -0.5, window, splits,
                     floats.data_ptr(), counters.data_ptr(), stream)
        assert rc == 0, lib.dinfer_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, ref), seed
    # beyond the fixed array: refused with a message, nothing launched
    rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), cache.data_ptr(), table.data_ptr(),
            table.shape[1], cu.data_ptr(), seq.data_ptr(), 4096, 64, 8, 128, 16, 0.1, 0, 32, stream)
    assert rc != 0 and b"fixed array" in lib.dinfer_last_error()
    # arguments the kernel does not take are refused before anything is queued
    rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), cache.data_ptr(), table.data_ptr(),
            table.shape[1], cu.data_ptr(), seq.data_ptr(), 2, 12, 1, 48, 4, 0.1, 0, 4, stream)
    assert rc != 0 and b"not supported" in lib.dinfer_last_error()
    torch.cuda.synchronize()
