"""Wrapper of the tcgen05 / TMA matrix product (bfloat16 operands, f32 accumulation in tensor memory)."""
from __future__ import annotations

from ctypes import c_int, c_int64, c_void_p
from typing import Optional

import torch

from .lib import KernelError, check, ptr, require_cuda, stream_handle
from .ops import _fn

NUM_SMS = 148
DECODE_MAX_TOKENS = 64          # up to here the operands are swapped (weight rows fill the tile)
MAX_SPLITS = 8                  # the portable cluster size

# Per device: the status word the tcgen05 kernels set when a bounded wait runs out.
_STATE = {}


def _state(device):
    st = _STATE.get(device)
    if st is None:
        st = {"status": torch.zeros(1, dtype=torch.int32, device=device)}
        _STATE[device] = st
    return st


def device_status(device=None) -> int:
    """The status word of the tcgen05 kernels (0 = fine).  Reading it synchronizes."""
    device = torch.device(device or torch.cuda.current_device())
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    st = _STATE.get(device)
    return int(st["status"].item()) if st else 0


def check_status(device=None) -> None:
    code = device_status(device)
    if code:
        raise KernelError(f"a tcgen05 kernel gave up a bounded wait (status {code}: 1 = producer waiting for a free "
                          f"stage, 2 = MMA waiting for a tile, 3 = epilogue waiting for the accumulator)")


def supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """bfloat16 operands whose rows TMA can address: K and the row strides multiples of 8 elements."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def decode_splits(tokens: int, N: int, K: int) -> int:
    """K splits of the decode orientation: one wave of CTAs (three fit an SM up to 16 tokens, two
    beyond), at least eight 64-wide K blocks per CTA, at most ``MAX_SPLITS`` (the CTAs of a tile are
    one thread-block cluster)."""
    tiles = (N + 127) // 128
    k_blocks = (K + 63) // 64
    slots = 3 * NUM_SMS if tokens <= 16 else 2 * NUM_SMS - 16
    return max(1, min(slots // tiles, k_blocks // 8, MAX_SPLITS))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: Optional[int] = None,
            gated: bool = False) -> torch.Tensor:
    """out[tokens, N] = x[tokens, K] @ w[N, K]^T.  out: bfloat16 or float32, last axis contiguous.
    ``gated`` (at most ``DECODE_MAX_TOKENS`` rows): the rows of w are (gate, up) pairs and out is
    [tokens, N / 2] with out[t, j] = silu(x w_2j) * (x w_2j+1)."""
    require_cuda(x, w, out)
    if not supported(x, w):
        raise KernelError("gemm_tc: bfloat16 operands with K and row strides multiples of 8 and 16-byte aligned bases")
    tokens, K = x.shape
    N = w.shape[0]
    if gated and (tokens > DECODE_MAX_TOKENS or N % 2):
        raise KernelError("gemm_tc: the gated epilogue takes at most 64 rows and an even number of weight rows")
    if w.shape[1] != K or out.shape != (tokens, N // 2 if gated else N) or out.stride(1) != 1 \
            or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    st = _state(x.device)
    if tokens <= DECODE_MAX_TOKENS:
        splits = decode_splits(tokens, N, K) if splits is None else max(1, min(int(splits), MAX_SPLITS))
    else:
        splits = 1
    lib, f = _fn("gemm_tc", "dinfer_gemm_tc",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int,
                  c_void_p, c_void_p])
    check(lib, f(ptr(x), x.stride(0), ptr(w), w.stride(0), ptr(out), out.stride(0), int(out.dtype == torch.float32),
                 tokens, N, K, int(splits), int(bool(gated)), ptr(st["status"]), stream_handle()), "gemm_tc")
    return out
