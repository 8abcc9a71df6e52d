"""From logits rows to token ids, on the device.

One row per request that samples in this step.  All-greedy batches take the argmax kernel; anything
else goes through penalties (if any row has them) and the fused temperature / min_p / top-k / top-p
/ Philox inverse-CDF kernel (order as in models/qwen3/src/executor.rs:534-605).  The random number of
a row depends only on the request's seed and on how many tokens it has produced
(crates/core/src/sampler.rs:84,183-191), never on its place in the batch.
"""
from __future__ import annotations

from ctypes import c_int, c_int64, c_void_p
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels.lib import check, ptr, stream_handle
from ..kernels.ops import _fn
from .params import SamplingParams


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise ValueError("argmax: logits must be float32 with a contiguous last axis")
    if out is None:
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
    lib, f = _fn("sampling", "dinfer_argmax", [c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p])
    check(lib, f(ptr(logits), logits.stride(0), ptr(out), R, V, stream_handle()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, seeds: torch.Tensor, offsets: torch.Tensor,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           min_p: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """temperature/top_p/min_p float32 [R], top_k int32 [R], seeds/offsets int64 [R] (bit patterns of uint64)."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise ValueError("sample: logits must be float32 with a contiguous last axis")
    if out is None:
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
    lib, f = _fn("sampling", "dinfer_sample",
                 [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_int, c_void_p])
    check(lib, f(ptr(logits), logits.stride(0), ptr(temperature), ptr(top_k), ptr(top_p), ptr(min_p),
                 ptr(seeds), ptr(offsets), ptr(out), R, V, stream_handle()), "sample")
    return out


def apply_penalties(logits: torch.Tensor, ids: torch.Tensor, offsets: torch.Tensor, prompt_len: torch.Tensor,
                    rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> torch.Tensor:
    """In place on ``logits``; history of row b is ids[offsets[b]:offsets[b+1]], prompt first."""
    R, V = logits.shape
    lib, f = _fn("sampling", "dinfer_penalties",
                 [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                  c_void_p])
    check(lib, f(ptr(logits), logits.stride(0), ptr(ids), ptr(offsets), ptr(prompt_len), ptr(rep), ptr(freq),
                 ptr(pres), R, V, stream_handle()), "penalties")
    return logits


def logit_bias(logits: torch.Tensor, rows: torch.Tensor, ids: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """In place: logits[rows[i], ids[i]] += bias[i] (int32, int32, float32 [n]; a pair appears once)."""
    R, V = logits.shape
    lib, f = _fn("sampling", "dinfer_logit_bias", [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    check(lib, f(ptr(logits), logits.stride(0), ptr(rows), ptr(ids), ptr(bias), rows.numel(), V, stream_handle()),
          "logit_bias")
    return logits


def logprobs(logits: torch.Tensor, chosen: torch.Tensor, k: int):
    """(ids int32 [R, k+1], logprobs float32 [R, k+1], rank int32 [R]) under log_softmax of ``logits``: column 0
    the chosen token, then the k most likely in descending order (ties to the lower id); rank = tokens strictly
    more likely than the chosen one."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or chosen.dtype != torch.int32 or chosen.numel() != R:
        raise ValueError("logprobs: logits float32 [R, V] with a contiguous last axis, chosen int32 [R]")
    ids = torch.empty((R, k + 1), dtype=torch.int32, device=logits.device)
    lp = torch.empty((R, k + 1), dtype=torch.float32, device=logits.device)
    rank = torch.empty(R, dtype=torch.int32, device=logits.device)
    lib, f = _fn("sampling", "dinfer_logprobs",
                 [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    check(lib, f(ptr(logits), logits.stride(0), ptr(chosen), int(k), ptr(ids), ptr(lp), ptr(rank), R, V,
                 stream_handle()), "logprobs")
    return ids, lp, rank


def _u64(x: int) -> int:
    x &= 0xFFFFFFFFFFFFFFFF
    return x - (1 << 64) if x >= (1 << 63) else x


class Sampler:
    """Builds the per-row columns on the host in pinned memory, uploads them in one copy and launches the
    kernels."""

    RING = 4

    def __init__(self, device):
        self.device = device
        self.last_logprobs = None       # (ids, logprobs, rank) of the last call, if any of its rows asked
        self._slots: List[dict] = []
        self._turn = 0
        self._rows = 0

    def _staging(self, rows: int) -> dict:
        """Pinned and device buffers of 32 bytes a row (a small ring: a buffer is rewritten only after its
        last copy has left it), with the views of their columns made once."""
        if rows > self._rows:
            cap = self._rows = max(64, 2 * rows)
            pin = torch.device(self.device).type == "cuda"
            self._slots = []
            for _ in range(self.RING):
                host = torch.empty(32 * cap, dtype=torch.uint8, pin_memory=pin)
                dev = torch.empty(32 * cap, dtype=torch.uint8, device=self.device)
                h = host.numpy()
                base = dev.data_ptr()
                self._slots.append(dict(
                    host=host, dev=dev, event=None,
                    # columns: seeds, offsets (int64), temperature, top_p, min_p (float32), top_k (int32)
                    i64=h[:16 * cap].view(np.int64).reshape(2, cap),
                    f32=h[16 * cap:28 * cap].view(np.float32).reshape(3, cap),
                    i32=h[28 * cap:32 * cap].view(np.int32),
                    seeds=base, offsets=base + 8 * cap, temperature=base + 16 * cap, top_p=base + 20 * cap,
                    min_p=base + 24 * cap, top_k=base + 28 * cap))
        k = self._turn
        self._turn = (k + 1) % self.RING
        slot = self._slots[k]
        if slot["event"] is not None:
            slot["event"].synchronize()
        return slot

    def __call__(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
                 num_generated: Sequence[int], histories: Optional[Sequence[tuple]] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Order: logit_bias -> penalties -> temperature -> min_p -> top-k -> top-p -> sample.
        ``histories[i] = (prompt_ids, output_ids)`` is needed only for rows with penalties.
        Returns int32 [R] on the device (``out`` if given); ``self.last_logprobs`` holds the log-probabilities
        if a row asked for them."""
        R, V = logits.shape
        raw = logits
        self.last_logprobs = None
        want_lp = [p.logprobs for p in params if p.logprobs is not None]
        if any(p.logit_bias for p in params):
            logits = logits.clone()
            rows_, ids_, vals_ = [], [], []
            for i, p in enumerate(params):
                for t, v in p.logit_bias.items():
                    rows_.append(i); ids_.append(int(t)); vals_.append(float(v))
            dev = self.device
            logit_bias(logits, torch.tensor(rows_, dtype=torch.int32, device=dev),
                       torch.tensor(ids_, dtype=torch.int32, device=dev),
                       torch.tensor(vals_, dtype=torch.float32, device=dev))
        toks = self._sample(logits, raw, params, seeds, num_generated, histories, out)
        if want_lp:
            # from the logits as the model gave them (models/qwen3/src/executor.rs:7,606-635)
            self.last_logprobs = logprobs(raw, toks, max(want_lp))
        return toks

    def _sample(self, logits, raw, params, seeds, num_generated, histories, out) -> torch.Tensor:
        R, V = logits.shape
        if all(p.is_greedy and not p.has_penalties for p in params):
            return argmax(logits, out)
        if any(p.has_penalties for p in params):
            if logits is raw:
                logits = logits.clone()
            flat: List[int] = []
            offs, plen = [0], []
            for i, p in enumerate(params):
                pr, ou = histories[i] if (histories and p.has_penalties) else ((), ())
                flat.extend(pr)
                flat.extend(ou)
                offs.append(len(flat))
                plen.append(len(pr))
            dev = self.device
            apply_penalties(
                logits, torch.tensor(flat or [0], dtype=torch.int32, device=dev),
                torch.tensor(offs, dtype=torch.int32, device=dev), torch.tensor(plen, dtype=torch.int32, device=dev),
                torch.tensor([p.repetition_penalty for p in params], dtype=torch.float32, device=dev),
                torch.tensor([p.frequency_penalty for p in params], dtype=torch.float32, device=dev),
                torch.tensor([p.presence_penalty for p in params], dtype=torch.float32, device=dev))
        if logits.dtype != torch.float32 or logits.stride(1) != 1:
            raise ValueError("sample: logits must be float32 with a contiguous last axis")
        slot = self._staging(R)
        i64, f32, i32 = slot["i64"], slot["f32"], slot["i32"]
        for i, p in enumerate(params):
            f32[0, i], f32[1, i], f32[2, i] = p.temperature, p.top_p, p.min_p
            i32[i] = p.top_k
            i64[0, i], i64[1, i] = _u64(seeds[i]), _u64(num_generated[i])
        slot["dev"].copy_(slot["host"], non_blocking=True)
        if slot["dev"].is_cuda:
            ev = slot["event"] or torch.cuda.Event()
            ev.record()
            slot["event"] = ev
        if out is None:
            out = torch.empty(R, dtype=torch.int32, device=logits.device)
        lib, f = _fn("sampling", "dinfer_sample",
                     [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_int, c_int, c_void_p])
        check(lib, f(ptr(logits), logits.stride(0), slot["temperature"], slot["top_k"], slot["top_p"], slot["min_p"],
                     slot["seeds"], slot["offsets"], ptr(out), R, V, stream_handle()), "sample")
        return out
