"""Typed Python wrappers over the C ABI of the kernel libraries.

Each wrapper checks what the kernel cannot (device, dtype, contiguity of the last axis), passes
explicit strides and the live token count, and launches on torch's current stream.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from .lib import KernelError, check, dtype_code, library, ptr, require_cuda, stream_handle

_sigs_done = set()


def _fn(libname: str, fname: str, argtypes):
    lib = library(libname)
    f = getattr(lib, fname)
    if (libname, fname) not in _sigs_done:
        f.argtypes = argtypes
        f.restype = c_int
        _sigs_done.add((libname, fname))
    return lib, f


def _rows_contiguous(t: torch.Tensor, what: str) -> None:
    if t.dim() < 1 or t.stride(-1) != 1:
        raise KernelError(f"{what}: last axis must be contiguous")


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
              prev: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] * scale into the f32 residual stream.  With ``prev`` (int32 [rows], the tokens
    the previous step sampled) an id -(r + 1) stands for prev[r]."""
    require_cuda(ids, table, out)
    T, h = out.shape
    if ids.dtype != torch.int32 or out.dtype != torch.float32 or not out.is_contiguous() \
            or not table.is_contiguous() or table.shape[1] != h or ids.numel() != T:
        raise KernelError("embedding: ids int32 [T], table [V, h] contiguous, out f32 [T, h] contiguous")
    if prev is not None:
        require_cuda(prev)
        if prev.dtype != torch.int32 or prev.dim() != 1 or not prev.is_contiguous():
            raise KernelError("embedding: prev int32 [rows] contiguous")
    lib, f = _fn("elementwise", "dinfer_embedding",
                 [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    check(lib, f(ptr(ids), ptr(prev) if prev is not None else None, prev.numel() if prev is not None else 0,
                 ptr(table), ptr(out), T, h, table.shape[0], dtype_code(table.dtype), float(scale), stream_handle()),
          "embedding")
    return out


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x = cap * tanh(x / cap) in place (float32, contiguous): logits with a soft cap."""
    require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous() or not cap > 0:
        raise KernelError("softcap: contiguous float32 values and a positive cap")
    lib, f = _fn("elementwise", "dinfer_softcap", [c_void_p, c_int64, c_float, c_void_p])
    check(lib, f(ptr(x), x.numel(), float(cap), stream_handle()), "softcap")
    return x


def rmsnorm(residual: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = rmsnorm(residual[src] + delta[src]) * weight, src = rows[r] or r; the sum is written
    back to ``residual`` when ``delta`` is given and ``rows`` is not."""
    require_cuda(residual, weight, out, delta, rows)
    h = residual.shape[-1]
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError("rmsnorm: residual must be contiguous float32")
    if not out.is_contiguous() or out.shape[-1] != h or weight.numel() != h or not weight.is_contiguous():
        raise KernelError("rmsnorm: out [R, h] contiguous, weight [h]")
    if delta is not None and (delta.dtype != out.dtype or delta.shape != residual.shape or not delta.is_contiguous()):
        raise KernelError("rmsnorm: delta must have the residual's shape and the output's dtype")
    if rows is not None:
        if rows.dtype != torch.int32 or rows.numel() != out.shape[0]:
            raise KernelError("rmsnorm: rows must be int32 [R]")
        n = rows.numel()
    else:
        n = residual.shape[0]
        if out.shape[0] != n:
            raise KernelError("rmsnorm: out must have the residual's row count")
    lib, f = _fn("norm", "dinfer_rmsnorm",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p])
    check(lib, f(ptr(residual), ptr(delta), ptr(rows), ptr(weight), ptr(out), n, h, float(eps),
                 dtype_code(out.dtype), dtype_code(weight.dtype), stream_handle()), "rmsnorm")
    return out


def rmsnorm_plain(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    require_cuda(x, weight, out)
    h = x.shape[-1]
    if not x.is_contiguous() or not out.is_contiguous() or out.shape != x.shape or out.dtype != x.dtype \
            or weight.numel() != h:
        raise KernelError("rmsnorm_plain: x, out contiguous of one shape and dtype; weight [h]")
    lib, f = _fn("norm", "dinfer_rmsnorm_plain",
                 [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), ptr(weight), ptr(out), x.numel() // h, h, float(eps), dtype_code(x.dtype),
                 dtype_code(weight.dtype), stream_handle()), "rmsnorm_plain")
    return out


def silu_mul(x: torch.Tensor, out: torch.Tensor, pairs: bool = False) -> torch.Tensor:
    """out[t, i] = silu(gate_i) * up_i for x [T, 2I] that holds gate and up as halves (gate_i = x[t, i],
    up_i = x[t, I + i]) or, with ``pairs``, side by side (gate_i = x[t, 2i], up_i = x[t, 2i + 1])."""
    require_cuda(x, out)
    _rows_contiguous(x, "silu_mul")
    T, two_i = x.shape
    inter = two_i // 2
    if two_i % 2 or out.shape != (T, inter) or not out.is_contiguous() or out.dtype != x.dtype:
        raise KernelError("silu_mul: x [T, 2I], out [T, I] contiguous, same dtype")
    lib, f = _fn("elementwise", "dinfer_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_void_p])
    check(lib, f(ptr(x), ptr(out), T, inter, x.stride(0), dtype_code(x.dtype), int(bool(pairs)), stream_handle()),
          "silu_mul")
    return out


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out[t, :] += bias, in place (a view with a row stride is fine)."""
    require_cuda(out, bias)
    _rows_contiguous(out, "add_bias")
    if out.dim() != 2 or bias.dim() != 1 or bias.numel() != out.shape[1] or not bias.is_contiguous():
        raise KernelError("add_bias: out [T, N], bias [N]")
    lib, f = _fn("elementwise", "dinfer_add_bias", [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(out), out.stride(0), ptr(bias), out.shape[0], out.shape[1], dtype_code(out.dtype),
                 dtype_code(bias.dtype), stream_handle()), "add_bias")
    return out


def cast(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    require_cuda(src, dst)
    if not src.is_contiguous() or not dst.is_contiguous() or src.numel() != dst.numel():
        raise KernelError("cast: contiguous tensors of one length")
    lib, f = _fn("elementwise", "dinfer_cast", [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p])
    check(lib, f(ptr(src), ptr(dst), src.numel(), dtype_code(src.dtype), dtype_code(dst.dtype),
                 stream_handle()), "cast")
    return dst


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T, 32-bit multiply-adds on the CUDA cores; each operand f32 or bf16."""
    require_cuda(a, w, out)
    for t, n in ((a, "a"), (w, "w"), (out, "out")):
        if t.dim() != 2:
            raise KernelError(f"gemm_f32: {n} must be 2-D")
        _rows_contiguous(t, "gemm_f32 " + n)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not agree")
    lib, f = _fn("gemm_f32", "dinfer_gemm_f32",
                 [c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int,
                  c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(a), a.stride(0), dtype_code(a.dtype), ptr(w), w.stride(0), dtype_code(w.dtype),
                 ptr(out), out.stride(0), dtype_code(out.dtype), M, N, K, stream_handle()), "gemm_f32")
    return out


def qk_post(qkv: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
            eps: float, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
            cos_sin: Optional[torch.Tensor], cache: Optional[torch.Tensor],
            slots: Optional[torch.Tensor], block_size: int, interleaved: bool = False) -> None:
    """Per-head RMSNorm of q and k, rotation (element i with i + rot/2, or with ``interleaved`` element 2i with
    2i + 1), write-back in place, k and v into the paged cache."""
    require_cuda(qkv, positions, q_weight, k_weight, cos_sin, cache, slots)
    _rows_contiguous(qkv, "qk_post")
    T = qkv.shape[0]
    if positions.dtype != torch.int32 or positions.numel() != T:
        raise KernelError("qk_post: positions int32 [T]")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qk_post: q and k norm weights come together")
    w_dt = q_weight.dtype if q_weight is not None else torch.float32
    if q_weight is not None and (q_weight.numel() != head_dim or k_weight.numel() != head_dim
                                 or k_weight.dtype != w_dt):
        raise KernelError("qk_post: norm weights must be [head_dim] of one dtype")
    rot = 0
    if cos_sin is not None:
        if cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous() or cos_sin.dim() != 2:
            raise KernelError("qk_post: angle table must be contiguous float32 [max_pos, rot]")
        rot = cos_sin.shape[1]
    if cache is not None:
        if cache.dtype != qkv.dtype or not cache.is_contiguous() or slots is None or slots.dtype != torch.int32 \
                or slots.numel() != T:
            raise KernelError("qk_post: cache of the activations' dtype, contiguous; slots int32 [T]")
        if tuple(cache.shape[1:]) != (2, num_kv_heads, block_size, head_dim):
            raise KernelError(f"qk_post: cache shape {tuple(cache.shape)} is not [blocks, 2, {num_kv_heads}, "
                              f"{block_size}, {head_dim}]")
    lib, f = _fn("qk_post", "dinfer_qk_post_styled",
                 [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    check(lib, f(ptr(qkv), qkv.stride(0), ptr(positions), ptr(q_weight), ptr(k_weight), float(eps),
                 ptr(cos_sin), rot, int(bool(interleaved)), ptr(cache), ptr(slots), block_size, T, num_heads, num_kv_heads,
                 head_dim, dtype_code(qkv.dtype), dtype_code(w_dt), stream_handle()), "qk_post")


def attention_generic(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      cu_seqlens: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int,
                      head_dim: int, scale: float, window: int = 0) -> torch.Tensor:
    """Paged causal attention, plain arithmetic, any head size.  ``q`` may be a strided view (for
    instance the q columns of the qkv rows)."""
    require_cuda(q, out, cache, block_table, cu_seqlens, positions)
    _rows_contiguous(q, "attention q")
    _rows_contiguous(out, "attention out")
    T = q.shape[0]
    B = cu_seqlens.numel() - 1
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, out and cache must have one dtype")
    for t, n in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (positions, "positions")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"attention: {n} must be contiguous int32")
    if block_table.dim() != 2 or block_table.shape[0] < B or positions.numel() != T:
        raise KernelError("attention: block_table [B, max_blocks], positions [T]")
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim \
            or not cache.is_contiguous():
        raise KernelError(f"attention: cache shape {tuple(cache.shape)} is not [blocks, 2, Hkv, block, D]")
    lib, f = _fn("attention_generic", "dinfer_attention_generic",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p])
    check(lib, f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(cache), ptr(block_table),
                 block_table.shape[1], ptr(cu_seqlens), ptr(positions), T, B, num_heads, num_kv_heads,
                 head_dim, cache.shape[3], float(scale), int(window), dtype_code(q.dtype), stream_handle()),
          "attention_generic")
    return out
