"""Grouped-query attention over the paged cache: the mixer of Qwen3 and of anything else that is
q/k/v projections, an optional per-head RMSNorm of q and k, a position encoding, causal softmax
attention (optionally over a window) and an output projection.

Data flow of one step (models/qwen3/src/model.rs:141-172,212-313):
  qkv = x Wqkv^T                       one fused product, rows laid out q heads | k heads | v heads
  q, k <- rope(headnorm(q, k)); k, v -> cache      one kernel, in place
  o = softmax(q k^T * scale + mask) v              over the cache, through the block table
  y = o Wo^T
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..kernels import attention_ops, ops
from .base import (MIXERS, POSITION_ENCODINGS, BuildEnv, CacheBinding, KvCacheNeed, Mixer, StepContext,
                   build_part)
from .linear import Linear
from .spec import PartSpec, TensorDecl


@MIXERS.register("gqa_attention")
class GQAttention(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``qk_norm`` (bool), ``eps``,
    ``position`` (a PartSpec), optional ``window``, ``scale``, ``bias`` (bool: the four projections have a bias,
    named like their weights with ``.bias``), and the tensor names ``q_proj``, ``k_proj``, ``v_proj``, ``o_proj``,
    ``q_norm``, ``k_norm`` (after the prefix)."""

    def __init__(self, params, env: BuildEnv, prefix=""):
        super().__init__(params, env, prefix)
        p = self.params
        self.hidden = env.hidden_size
        self.H = int(p["num_heads"])
        self.Hkv = int(p["num_kv_heads"])
        self.D = int(p["head_dim"])
        if self.H % self.Hkv:
            raise ValueError(f"heads {self.H} not divisible by kv heads {self.Hkv}")
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("eps", 1e-6))
        self.window = p.get("window")
        self.page_size = p.get("cache_block_size")           # None: the engine's page size
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.D)))
        self.bias = bool(p.get("bias", False))
        pos: PartSpec = p.get("position") or PartSpec("none")
        self.position = build_part(POSITION_ENCODINGS, pos, env, prefix)
        n = lambda key, default: prefix + p.get(key, default)
        self.names = {
            "q": n("q_proj", "q_proj.weight"), "k": n("k_proj", "k_proj.weight"),
            "v": n("v_proj", "v_proj.weight"), "o": n("o_proj", "o_proj.weight"),
            "qn": n("q_norm", "q_norm.weight"), "kn": n("k_norm", "k_norm.weight"),
        }
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.q_norm_w = self.k_norm_w = None

    def declare(self) -> List[TensorDecl]:
        H, Hkv, D, h = self.H, self.Hkv, self.D, self.hidden
        d = [TensorDecl(self.names["q"], (H * D, h)), TensorDecl(self.names["k"], (Hkv * D, h)),
             TensorDecl(self.names["v"], (Hkv * D, h)), TensorDecl(self.names["o"], (h, H * D))]
        if self.qk_norm:
            d += [TensorDecl(self.names["qn"], (D,), init="ones"), TensorDecl(self.names["kn"], (D,), init="ones")]
        if self.bias:
            d += [TensorDecl(self._bias_name(x), (n,)) for x, n in (("q", H * D), ("k", Hkv * D), ("v", Hkv * D), ("o", h))]
        return d

    def _bias_name(self, which: str) -> str:
        name = self.names[which]
        return (name[:-len(".weight")] if name.endswith(".weight") else name) + ".bias"

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        q, k, v = (tensors[self.names[x]] for x in ("q", "k", "v"))
        dt = torch.float32 if any(t.dtype == torch.float32 for t in (q, k, v)) else q.dtype
        # q, k, v rows stacked once at load into one [(H + 2 Hkv) D, h] matrix (model.rs:141-164)
        qkv_bias = o_bias = None
        if self.bias:
            qkv_bias = torch.cat([tensors[self._bias_name(x)].to(dt) for x in ("q", "k", "v")])
            o_bias = tensors[self._bias_name("o")]
        self.qkv = Linear(torch.cat([q.to(dt), k.to(dt), v.to(dt)], dim=0), qkv_bias)
        self.o = Linear(tensors[self.names["o"]], o_bias)
        if self.qk_norm:
            self.q_norm_w = tensors[self.names["qn"]].contiguous()
            self.k_norm_w = tensors[self.names["kn"]].to(self.q_norm_w.dtype).contiguous()

    def cache_need(self):
        return KvCacheNeed(self.Hkv, self.D, self.window, int(self.page_size) if self.page_size else None)

    def kernel_libraries(self):
        att = ["attention_generic"]
        if attention_ops.tc_supported(self.env.act_dtype, self.D, self.H // self.Hkv):
            att = ["attention_tc"]
            if self.D in (64, 128):
                att += ["attention_decode", "attention_umma", "attention_umma64"]
        return ["qk_post"] + att + self.qkv.kernel_libraries() + self.o.kernel_libraries()

    def takes_half_normed(self, rows: int) -> bool:
        return self.qkv.fuses_norm(rows, self.env.act_dtype)

    def adds_into_residual(self, rows: int) -> bool:
        return self.o.fuses_norm(rows, self.env.act_dtype)

    def forward(self, x, ctx: StepContext, cache: CacheBinding, sink=None):
        H, Hkv, D = self.H, self.Hkv, self.D
        g = ctx.groups[cache.group]
        qkv = self.qkv(x)
        kv = cache.kv if cache.write else None
        table = self.position.fused_table()
        if self.position.fused:
            ops.qk_post(qkv, ctx.positions, H, Hkv, D, self.eps, self.q_norm_w, self.k_norm_w, table,
                        kv, g.slot_mapping, g.block_size, interleaved=getattr(self.position, "interleaved", False))
        else:
            if self.qk_norm:
                ops.qk_post(qkv, ctx.positions, H, Hkv, D, self.eps, self.q_norm_w, self.k_norm_w, None,
                            None, None, g.block_size)
            T = qkv.shape[0]
            self.position.apply(qkv[:, :H * D].unflatten(1, (H, D)),
                                qkv[:, H * D:(H + Hkv) * D].unflatten(1, (Hkv, D)), ctx)
            if kv is not None:
                ops.qk_post(qkv, ctx.positions, H, Hkv, D, self.eps, None, None, None, kv,
                            g.slot_mapping, g.block_size)
        out = torch.empty((qkv.shape[0], H * D), dtype=qkv.dtype, device=qkv.device)
        self.attend(qkv[:, :H * D], out, cache.kv, g, ctx)
        if sink is not None:                               # (residual, the norm behind this mixer)
            return self.o.into_residual(out, sink[0], sink[1])
        return self.o(out)

    def attend(self, q, out, kv, g, ctx: StepContext) -> None:
        """Tensor-core kernels where they take the head size (bfloat16; 32, 64, 128), else the
        plain-arithmetic kernel, which takes every size."""
        window = int(self.window or 0)
        if attention_ops.tc_supported(q.dtype, self.D, self.H // self.Hkv):
            splits = ctx.decode_splits or attention_ops.decode_splits(ctx.num_reqs, self.Hkv, ctx.max_seq_len)
            tc_decode = ctx.any_decode
            if ctx.any_decode and attention_ops.decode_supported(q.dtype, self.D, self.H // self.Hkv, g.block_size):
                # decoded tokens: the kernel made for them (keys on the tile's rows, in-kernel fold)
                attention_ops.attention_decode(q, out, kv, g.block_table, ctx.cu_seqlens, ctx.seq_lens, self.H,
                                               self.Hkv, self.D, self.scale, window, splits)
                tc_decode = False
            tc_prefill = ctx.any_prefill
            if ctx.any_prefill and attention_ops.umma_supported(q.dtype, self.D, self.H // self.Hkv, g.block_size):
                # prompt portions: tcgen05 / TMEM / TMA
                key = ("attention_umma", self.H, self.Hkv, self.D)
                shape = ctx.derived.get(key)
                if shape is None:
                    cu = ctx.cu_seqlens_host
                    lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
                    group = self.H // self.Hkv
                    shape = ctx.derived[key] = (
                        attention_ops.umma_key_splits(lens or [ctx.max_q_len], group, self.Hkv, self.D, ctx.max_seq_len),
                        attention_ops.umma_pair_bound(lens, group) if lens else 0)
                if ((ctx.max_prefill_seq_len or ctx.max_seq_len) <= attention_ops.UMMA_SHORT_CONTEXT
                        and attention_ops.umma64_supported(q.dtype, self.D, self.H // self.Hkv, g.block_size)):
                    attention_ops.attention_umma64(q, out, kv, g.block_table, ctx.cu_seqlens, ctx.seq_lens, self.H,
                                                   self.Hkv, self.D, self.scale, window, ctx.max_q_len, shape[1])
                else:
                    attention_ops.attention_umma(q, out, kv, g.block_table, ctx.cu_seqlens, ctx.seq_lens, self.H,
                                                 self.Hkv, self.D, self.scale, window, ctx.max_q_len, shape[0], shape[1])
                tc_prefill = False
            if tc_decode or tc_prefill:
                attention_ops.attention_tc(q, out, kv, g.block_table, ctx.cu_seqlens, ctx.seq_lens, self.H,
                                           self.Hkv, self.D, self.scale, window, ctx.max_q_len, tc_decode,
                                           tc_prefill, splits)
        else:
            ops.attention_generic(q, out, kv, g.block_table, ctx.cu_seqlens, ctx.positions, self.H, self.Hkv,
                                  self.D, self.scale, window)
