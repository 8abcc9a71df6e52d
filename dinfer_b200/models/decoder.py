"""The one model class: a decoder put together from a ``ModelSpec``.

embedding -> the schedule's layer runs over a 32-bit residual stream -> final norm at the wanted
rows -> head -> f32 logits (models/qwen3/src/model.rs:684-853 for the order of operations).
Which parts a layer has, and in which order layers run, is data in the spec.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..parts import attention, block, mlp, norm, rope  # noqa: F401  (register the built-in parts)
from ..parts.base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, BuildEnv, CacheBinding, ResidualStream,
                          StepContext, build_part)
from ..parts.linear import Linear
from ..parts.spec import ModelSpec, TensorDecl


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        spec.check()
        if env.hidden_size != spec.hidden_size:
            raise ValueError("BuildEnv.hidden_size differs from the spec's")
        self.spec, self.env = spec, env
        self.blocks = []
        for ls in spec.layers:
            mixer = build_part(MIXERS, ls.mixer, env, ls.prefix)
            mnorm = build_part(NORMS, ls.mixer_norm, env, ls.prefix)
            ffn = build_part(FEED_FORWARDS, ls.feed_forward, env, ls.prefix)
            fnorm = build_part(NORMS, ls.feed_forward_norm, env, ls.prefix)
            self.blocks.append(BLOCKS.get(ls.block)(mixer, mnorm, ffn, fnorm))
        self.final_norm = build_part(NORMS, spec.final_norm, env, "")
        self.embedding: Optional[torch.Tensor] = None
        self.lm_head: Optional[Linear] = None

    # ---- weights
    def declarations(self) -> List[TensorDecl]:
        s = self.spec
        d = [TensorDecl(s.embedding_tensor, (s.vocab_size, s.hidden_size))]
        for b in self.blocks:
            for p in b.parts():
                d += p.declare()
        d += self.final_norm.declare()
        # the head falls back to the embedding table only when the configuration ties them
        # (models/qwen3/src/model.rs:487-496)
        d.append(TensorDecl(s.lm_head_tensor, (s.vocab_size, s.hidden_size), optional=s.tie_word_embeddings))
        return d

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[s.embedding_tensor].contiguous()
        for b in self.blocks:
            for p in b.parts():
                p.bind(tensors)
        self.final_norm.bind(tensors)
        head = tensors.get(s.lm_head_tensor)
        self.lm_head = Linear(head if head is not None else self.embedding)

    def kernel_libraries(self) -> List[str]:
        libs = ["elementwise"] + self.lm_head.kernel_libraries() + self.final_norm.kernel_libraries()
        for b in self.blocks:
            for p in b.parts():
                libs += p.kernel_libraries()
        return list(dict.fromkeys(libs))

    # ---- caches
    def cache_needs(self) -> List[object]:
        """For each schedule entry: what its mixer keeps (None for an entry that reads another's)."""
        out = []
        for e in self.spec.schedule:
            out.append(None if e.cache_from is not None else self.blocks[e.layer].mixer.cache_need())
        return out

    def graph_capturable(self) -> bool:
        """Whether a step of this model can be captured in a CUDA graph: every mixer that keeps per-request state
        must say so (``Mixer.graph_capturable``); mixers without state always can."""
        from ..parts.base import StateNeed
        return all(not isinstance(b.mixer.cache_need(), StateNeed) or bool(b.mixer.graph_capturable) for b in self.blocks)

    def can_split_norms(self, rows: int) -> bool:
        """Whether some norm of the model can be taken apart for steps of this many rows."""
        from ..parts.block import norm_comes_apart
        order = [self.blocks[e.layer] for e in self.spec.schedule]
        for i, b in enumerate(order):
            if norm_comes_apart(b.mixer, b.feed_forward_norm, b.feed_forward, rows):
                return True
            if i + 1 < len(order) and norm_comes_apart(b.feed_forward, order[i + 1].mixer_norm, order[i + 1].mixer, rows):
                return True
        return False

    # ---- one step
    def forward(self, ids: torch.Tensor, ctx: StepContext, bindings: List[CacheBinding],
                logits_rows: torch.Tensor) -> torch.Tensor:
        """ids [T] int32 -> logits [R, V] float32 at the rows ``logits_rows`` [R] int32."""
        s = self.spec
        T = ids.numel()
        x = torch.empty((T, s.hidden_size), dtype=torch.float32, device=ids.device)
        ops.embedding(ids, self.embedding, x, prev=ctx.prev_tokens, scale=s.embedding_scale)
        stream = ResidualStream(x)
        order = [self.blocks[e.layer] for e in s.schedule]
        for i, (block, binding) in enumerate(zip(order, bindings)):
            block.forward(stream, ctx, binding, next_block=order[i + 1] if i + 1 < len(order) else None)
        if logits_rows.numel() == 0:
            return torch.empty((0, s.vocab_size), dtype=torch.float32, device=ids.device)
        f = self.final_norm.forward(stream.x, delta=stream.pending, rows=logits_rows)
        logits = self.lm_head(f, out_dtype=torch.float32)
        if s.logit_softcap > 0:
            ops.softcap(logits, s.logit_softcap)
        return logits
