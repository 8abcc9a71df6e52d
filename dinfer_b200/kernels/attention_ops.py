"""Wrapper of the tensor-core attention library (bfloat16; head sizes 32, 64, 128)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from .lib import KernelError, check, num_sms, ptr, require_cuda, stream_handle
from .ops import _fn

MAX_CLUSTER_SPLITS = 16         # key splits of the TMA decode kernel: one thread-block cluster
# The prompt attention has a kernel with 64-key tiles beside the one with 128-key tiles: steps whose longest
# request stays within this many tokens run the first (measured: it wins up to about 512 keys a row, at 1024
# the two meet, beyond that and behind long histories the second wins)
UMMA_SHORT_CONTEXT = 512


def tc_supported(dtype: torch.dtype, head_dim: int, group: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (32, 64, 128) and 1 <= group <= 16


def decode_splits(num_reqs: int, num_kv_heads: int, max_seq_len: int) -> int:
    """Key splits of the decode shape.  Two CTAs fit an SM: with few (request, kv head) pairs the
    splits fill those slots in one wave; with as many pairs as slots or more, splitting only adds
    partial sums to fold, so there is none.  Never more than a quarter of the 64-key tiles, at
    most 16 (the largest cluster)."""
    slots = 2 * num_sms()
    base = max(1, num_reqs * num_kv_heads)
    want = slots // base if base <= slots else 1
    tiles = max(1, (max_seq_len + 63) // 64)
    return max(1, min(want, max(1, tiles // 4), MAX_CLUSTER_SPLITS))


def decode_supported(dtype: torch.dtype, head_dim: int, group: int, block_size: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and 1 <= group <= 16
            and block_size > 0 and block_size & (block_size - 1) == 0)


# Scratch of the split-key decode kernel, per device: f32 partial sums and a block of counters that
# every launch leaves at zero.  Buffers are only ever replaced by larger ones and the old ones are
# kept alive, because a captured CUDA graph holds their addresses.  All launches that use it run on
# one stream (they must not overlap).
_SCRATCH = {}
_SCRATCH_KEEP = []


def _decode_scratch(device, n_floats: int, n_counters: int):
    cur = _SCRATCH.get(device)
    if cur is None or cur[0].numel() < n_floats or cur[1].numel() < n_counters:
        floats = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
        counters = torch.zeros(max(n_counters, 1 << 14), dtype=torch.int32, device=device)
        if cur is not None:
            _SCRATCH_KEEP.append(cur)
        cur = (floats, counters)
        _SCRATCH[device] = cur
    return cur


def attention_decode(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                     cu_seqlens: torch.Tensor, seq_lens: torch.Tensor, num_heads: int, num_kv_heads: int,
                     head_dim: int, scale: float, window: int, splits: int) -> torch.Tensor:
    """Attention of the requests that bring exactly one token (the others are skipped), keys split
    ``splits`` ways; the splits are folded inside the kernel."""
    require_cuda(q, out, cache, block_table, cu_seqlens, seq_lens)
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 only")
    if q.stride(-1) != 1 or out.stride(-1) != 1 or not cache.is_contiguous():
        raise KernelError("attention_decode: contiguous last axes and a contiguous cache")
    B = cu_seqlens.numel() - 1
    for t, n in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (seq_lens, "seq_lens")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"attention_decode: {n} must be contiguous int32")
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
        raise KernelError(f"attention_decode: cache shape {tuple(cache.shape)} is not [blocks, 2, Hkv, block, D]")
    if cache.shape[3] >= 8:
        # pages of at least 8 tokens: tiles by TMA through a tensor map over the cache, mbarrier ring;
        # the splits of a (request, kv head) are one thread-block cluster and fold through shared memory
        from . import gemm_ops
        status = gemm_ops._state(q.device)["status"]
        lib, f = _fn("attention_decode", "dinfer_attention_decode_tma",
                     [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p,
                      c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p])
        check(lib, f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(cache), cache.shape[0], ptr(block_table),
                     block_table.shape[1], ptr(cu_seqlens), ptr(seq_lens), B, num_heads, num_kv_heads, head_dim,
                     cache.shape[3], float(scale), int(window), min(int(splits), MAX_CLUSTER_SPLITS), ptr(status),
                     stream_handle()), "attention_decode_tma")
        return out
    floats = counters = None
    if splits > 1:
        floats, counters = _decode_scratch(q.device, B * num_heads * splits * (head_dim + 2), B * num_kv_heads)
    lib, f = _fn("attention_decode", "dinfer_attention_decode",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p])
    check(lib, f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(cache), ptr(block_table), block_table.shape[1],
                 ptr(cu_seqlens), ptr(seq_lens), B, num_heads, num_kv_heads, head_dim, cache.shape[3],
                 float(scale), int(window), int(splits), ptr(floats), ptr(counters), stream_handle()),
          "attention_decode")
    return out


def umma_supported(dtype: torch.dtype, head_dim: int, group: int, block_size: int) -> bool:
    """The tcgen05 prompt attention: bfloat16, head size 64 or 128, a group that divides 128,
    power-of-two pages of at least 8 tokens."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and group >= 1 and 128 % group == 0
            and block_size >= 8 and block_size & (block_size - 1) == 0)


_UMMA_CLUSTERS = {}


def umma_max_clusters(head_dim: int, key_splits: int) -> int:
    """Clusters of ``key_splits`` CTAs of the prompt attention that the device runs at a time (asked once)."""
    key = (torch.cuda.current_device(), head_dim, key_splits)
    if key not in _UMMA_CLUSTERS:
        lib, f = _fn("attention_umma", "dinfer_attention_umma_max_clusters", [c_int, c_int])
        n = f(head_dim, key_splits)
        if n < 0:
            msg = lib.dinfer_last_error()
            raise KernelError(f"attention_umma_max_clusters failed (code {-n}): {msg.decode('utf-8', 'replace') if msg else ''}")
        _UMMA_CLUSTERS[key] = n
    return _UMMA_CLUSTERS[key]


def umma64_supported(dtype: torch.dtype, head_dim: int, group: int, block_size: int) -> bool:
    """The 64-key-tile prompt attention: as ``umma_supported``, with pages of at most 64 tokens."""
    return umma_supported(dtype, head_dim, group, block_size) and block_size <= 64


def umma_pair_bound(portion_lens, group: int) -> int:
    """An upper bound of the 256-row tile pairs of a step's prompt portions, which the kernel's grid counts.  It
    holds for every way of spreading the same prompt tokens over the same places (a captured graph is replayed
    on portions of other lengths): places without tokens count as places, requests that bring one token (they
    belong to the decode kernel) do not."""
    tokens = sum(n for n in portion_lens if n != 1)
    places = sum(1 for n in portion_lens if n != 1)
    return max(1, (tokens * group + 255 * places) // 256)


def umma_key_splits(portion_lens, group: int, num_kv_heads: int, head_dim: int, max_seq_len: int) -> int:
    """How many CTAs share the keys of one 256-row tile pair of the prompt attention.  A CTA walks its
    128-key tiles one after the other, so a step with fewer tile pairs than SMs (one portion of 512
    tokens behind a long history: 64 pairs at 8 kv heads) leaves SMs idle while the others run long
    chains.  The keys are split as far as all clusters still run at the same time (a second wave
    would cost more than the shorter chains save), each CTA keeping at least four tiles of the
    longest request; at most 8 ways (the portable cluster size).  The count is an upper bound: in the
    kernel a pair with fewer key tiles is shared by fewer CTAs and the rest of its cluster leaves at
    once, so a graph captured for the longest request there may be costs a short one nothing.
    ``portion_lens``: tokens each request brings in this step (those with one token do not count)."""
    pairs = sum((n * group + 255) // 256 for n in portion_lens if n > 1) * num_kv_heads
    if pairs <= 0:
        return 1
    tiles = (max_seq_len + 127) // 128
    splits = 1
    while splits < 8 and tiles >= splits * 2 * 4 and pairs <= umma_max_clusters(head_dim, splits * 2):
        splits *= 2
    return splits


def attention_umma(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                   cu_seqlens: torch.Tensor, seq_lens: torch.Tensor, num_heads: int, num_kv_heads: int,
                   head_dim: int, scale: float, window: int, max_q_len: int, key_splits: int = 1,
                   pair_bound: int = 0) -> torch.Tensor:
    """Attention of the prompt portions of the batch (requests with more than one token; the others
    are skipped) on tcgen05 / TMEM / TMA.  ``q``: the [T, H*D] columns of the step's rows (a view with a
    row stride is fine).  ``key_splits``: see ``umma_key_splits``; ``pair_bound``: see ``umma_pair_bound``
    (0: every request is taken for the longest portion)."""
    _umma_launch(False, q, out, cache, block_table, cu_seqlens, seq_lens, num_heads, num_kv_heads, head_dim, scale,
                 window, max_q_len, key_splits, pair_bound)
    return out


def attention_umma64(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                     cu_seqlens: torch.Tensor, seq_lens: torch.Tensor, num_heads: int, num_kv_heads: int,
                     head_dim: int, scale: float, window: int, max_q_len: int, pair_bound: int = 0) -> torch.Tensor:
    """The same attention through the kernel with 64-key tiles (``UMMA_SHORT_CONTEXT``); no key split."""
    _umma_launch(True, q, out, cache, block_table, cu_seqlens, seq_lens, num_heads, num_kv_heads, head_dim, scale,
                 window, max_q_len, 1, pair_bound)
    return out


def _umma_launch(short, q, out, cache, block_table, cu_seqlens, seq_lens, num_heads, num_kv_heads, head_dim, scale,
                 window, max_q_len, key_splits, pair_bound) -> None:
    from . import gemm_ops
    require_cuda(q, out, cache, block_table, cu_seqlens, seq_lens)
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_umma: bfloat16 only")
    if q.stride(-1) != 1 or out.stride(-1) != 1 or not cache.is_contiguous():
        raise KernelError("attention_umma: contiguous last axes and a contiguous cache")
    B = cu_seqlens.numel() - 1
    for t, n in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (seq_lens, "seq_lens")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"attention_umma: {n} must be contiguous int32")
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
        raise KernelError(f"attention_umma: cache shape {tuple(cache.shape)} is not [blocks, 2, Hkv, block, D]")
    status = gemm_ops._state(q.device)["status"]
    head = (ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(cache), cache.shape[0], ptr(block_table),
            block_table.shape[1], ptr(cu_seqlens), ptr(seq_lens), q.shape[0], B, num_heads, num_kv_heads,
            head_dim, cache.shape[3], float(scale), int(window), int(max_q_len), int(pair_bound))
    types = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int]
    if short:
        lib, f = _fn("attention_umma64", "dinfer_attention_umma64", types + [c_void_p, c_void_p])
        check(lib, f(*head, ptr(status), stream_handle()), "attention_umma64")
    else:
        lib, f = _fn("attention_umma", "dinfer_attention_umma", types + [c_int, c_void_p, c_void_p])
        check(lib, f(*head, int(key_splits), ptr(status), stream_handle()), "attention_umma")


def attention_tc(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                 cu_seqlens: torch.Tensor, seq_lens: torch.Tensor, num_heads: int, num_kv_heads: int,
                 head_dim: int, scale: float, window: int, max_q_len: int, any_decode: bool,
                 any_prefill: bool, splits: int, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged causal attention on the tensor cores.  ``q`` / ``out``: rows with a contiguous last axis,
    head h at columns [h*D, (h+1)*D).  ``splits`` > 1 needs ``scratch`` (f32) of
    ``B * H * splits * (D + 2)`` elements; it is allocated here when not given."""
    require_cuda(q, out, cache, block_table, cu_seqlens, seq_lens)
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_tc: bfloat16 only")
    if q.stride(-1) != 1 or out.stride(-1) != 1 or not cache.is_contiguous():
        raise KernelError("attention_tc: contiguous last axes and a contiguous cache")
    B = cu_seqlens.numel() - 1
    for t, n in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (seq_lens, "seq_lens")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"attention_tc: {n} must be contiguous int32")
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
        raise KernelError(f"attention_tc: cache shape {tuple(cache.shape)} is not [blocks, 2, Hkv, block, D]")
    if not any_decode:
        splits = 1
    if splits > 1 and scratch is None:
        scratch = torch.empty(B * num_heads * splits * (head_dim + 2), dtype=torch.float32, device=q.device)
    if splits > 1 and (scratch.dtype != torch.float32 or scratch.numel() < B * num_heads * splits * (head_dim + 2)):
        raise KernelError("attention_tc: scratch too small")
    lib, f = _fn("attention_tc", "dinfer_attention_tc",
                 [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    check(lib, f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(cache), ptr(block_table), block_table.shape[1],
                 ptr(cu_seqlens), ptr(seq_lens), B, num_heads, num_kv_heads, head_dim, cache.shape[3],
                 float(scale), int(window), int(max_q_len), int(any_decode), int(any_prefill), int(splits),
                 ptr(scratch if splits > 1 else None), stream_handle()), "attention_tc")
    return out
