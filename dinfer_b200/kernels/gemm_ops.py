"""Wrapper of the tcgen05 / TMA matrix product (bfloat16 operands, f32 accumulation in tensor memory)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from .lib import KernelError, check, num_sms, ptr, require_cuda, stream_handle
from .ops import _fn

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


def _device(device=None) -> torch.device:
    device = torch.device(device if device is not None else torch.cuda.current_device())
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def device_status(device=None) -> int:
    """The status word of the kernels with bounded waits (0 = fine).  Reading it synchronizes."""
    st = _STATE.get(_device(device))
    return int(st["status"].item()) if st else 0


# what a kernel was waiting for when it gave up (the code it left in the status word)
STATUS_MEANING = {
    1: "matrix product: the TMA producer waited for a free shared-memory stage",
    2: "matrix product: the MMA thread waited for an operand tile (or a free accumulator)",
    3: "matrix product: the epilogue warps waited for the accumulator",
    11: "prompt attention: the TMA producer waited for a free K/V stage",
    12: "prompt attention: the MMA thread waited for the Q or the first K tiles",
    13: "prompt attention: the MMA thread waited for the softmax warps' P tile",
    14: "prompt attention: the MMA thread waited for a K or V tile",
    15: "prompt attention: the softmax warps waited for a score tile or for P V to finish",
    16: "prompt attention: the softmax warps waited for the last P V before writing the output",
    21: "decode attention: the TMA producer waited for a free stage",
    22: "decode attention: the compute warps waited for a key/value tile",
}


def describe_status(code: int) -> str:
    return STATUS_MEANING.get(int(code), "unknown code")


def check_status(device=None) -> None:
    """Raise if a kernel gave up one of its bounded waits.  The word stays set (every later check raises too)
    until ``reset_status``: after such a fault the step's results are not to be trusted."""
    code = device_status(device)
    if code:
        raise KernelError(f"a kernel gave up a bounded wait and returned early (status {code}: "
                          f"{describe_status(code)}); the results of that step are invalid")


def reset_status(device=None) -> int:
    """Clear the status word; returns the code it held."""
    st = _STATE.get(_device(device))
    if st is None:
        return 0
    code = int(st["status"].item())
    st["status"].zero_()
    return code


def wait_probe(polls: int = 1000, device=None) -> int:
    """Launch one CTA that allocates tensor memory and waits, with the products' own bounded wait cut down to
    ``polls`` polls, on an mbarrier nobody arrives at; it must give up, record code 2 in the status word, free its
    tensor memory and return.  Returns the status word after it (reading synchronizes).  For tests of the
    failure path; nothing in the engine calls it."""
    device = _device(device)
    st = _state(device)
    lib, f = _fn("gemm_tc", "dinfer_gemm_tc_wait_probe", [c_void_p, c_int, c_void_p])
    with torch.cuda.device(device):
        check(lib, f(ptr(st["status"]), int(polls), stream_handle()), "gemm_tc_wait_probe")
    return device_status(device)


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
    sms = num_sms()
    slots = 3 * sms if tokens <= 16 else 2 * sms - 16
    return max(1, min(slots // tiles, k_blocks // 8, MAX_SPLITS))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: Optional[int] = None,
            gated: bool = False, residual: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
            sums: Optional[torch.Tensor] = None, row_scale=None) -> torch.Tensor:
    """out[tokens, N] = x[tokens, K] @ w[N, K]^T.  out: bfloat16 or float32, last axis contiguous.

    ``gated`` (any number of rows): the rows of w are (gate, up) pairs, out is [tokens, N / 2],
    out[t, j] = silu(x w_2j) * (x w_2j+1).
    Epilogues of the decode orientation (at most ``DECODE_MAX_TOKENS`` rows):
      ``residual`` [tokens, N] f32 with ``norm_weight`` [N] and ``sums`` [parts, stride >= tokens] f32
        (``parts = residual_parts(...)``): the product is added into the residual, out gets the new
        residual times the norm weight, ``sums[p, t]`` the squares of row t summed over part p;
      ``row_scale = (sums, parts, size, eps)``: out[t] *= rsqrt(sum_p sums[p, t] / size + eps).
    """
    require_cuda(x, w, out)
    if not supported(x, w):
        raise KernelError("gemm_tc: bfloat16 operands with K and row strides multiples of 8 and 16-byte aligned bases")
    tokens, K = x.shape
    N = w.shape[0]
    if (residual is not None or row_scale is not None) and tokens > DECODE_MAX_TOKENS:
        raise KernelError("gemm_tc: the norm epilogues take at most 64 rows")
    if gated and (N % 2 or residual is not None):
        raise KernelError("gemm_tc: the gated epilogue needs an even number of weight rows and no residual")
    if w.shape[1] != K or out.shape != (tokens, N // 2 if gated else N) or out.stride(1) != 1 \
            or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    st = _state(x.device)
    if tokens <= DECODE_MAX_TOKENS:
        splits = decode_splits(tokens, N, K) if splits is None else max(1, min(int(splits), MAX_SPLITS))
    else:
        splits = 1
    r_ptr = nw_ptr = so_ptr = si_ptr = None
    ldr = nw_f32 = parts = stride = 0
    inv_size = eps = 0.0
    if residual is not None:
        require_cuda(residual, norm_weight, sums)
        if (residual.dtype != torch.float32 or residual.shape != (tokens, N) or residual.stride(1) != 1
                or norm_weight.shape != (N,) or not norm_weight.is_contiguous()
                or norm_weight.dtype not in (torch.bfloat16, torch.float32)
                or sums.dtype != torch.float32 or sums.dim() != 2 or sums.stride(1) != 1 or sums.shape[1] < tokens
                or sums.shape[0] < residual_parts(tokens, N, K, splits)):
            raise KernelError("gemm_tc: residual [tokens, N] f32, norm_weight [N], sums [parts, >= tokens] f32")
        r_ptr, ldr, nw_ptr, nw_f32 = ptr(residual), residual.stride(0), ptr(norm_weight), int(norm_weight.dtype == torch.float32)
        so_ptr, stride = ptr(sums), sums.stride(0)
    if row_scale is not None:
        s_in, parts, size, eps = row_scale
        require_cuda(s_in)
        if s_in.dtype != torch.float32 or s_in.dim() != 2 or s_in.stride(1) != 1 or s_in.shape[1] < tokens \
                or not (0 < parts <= s_in.shape[0]):
            raise KernelError("gemm_tc: row_scale sums [parts, >= tokens] f32")
        if residual is not None and s_in.stride(0) != stride:
            raise KernelError("gemm_tc: the sums read and written must have one row stride")
        si_ptr, stride, inv_size = ptr(s_in), s_in.stride(0), 1.0 / float(size)
    lib, f = _fn("gemm_tc", "dinfer_gemm_tc_fused",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int,
                  c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_float,
                  c_void_p, c_void_p])
    check(lib, f(ptr(x), x.stride(0), ptr(w), w.stride(0), ptr(out), out.stride(0), int(out.dtype == torch.float32),
                 tokens, N, K, int(splits), int(bool(gated)), r_ptr, ldr, nw_ptr, nw_f32, so_ptr, si_ptr, int(parts),
                 int(stride), float(inv_size), float(eps), ptr(st["status"]), stream_handle()), "gemm_tc")
    return out


def residual_parts(tokens: int, N: int, K: int, splits: Optional[int] = None) -> int:
    """Rows of the ``sums`` the residual epilogue writes for these sizes."""
    if splits is None:
        splits = decode_splits(tokens, N, K)
    lib, f = _fn("gemm_tc", "dinfer_gemm_tc_parts", [c_int, c_int, c_int, c_int])
    return int(f(tokens, N, K, int(splits)))

