"""Arrangements of a layer's four parts around the residual stream."""
from __future__ import annotations

from typing import Optional

from .base import BLOCKS, Block, CacheBinding, ResidualStream, StepContext
from .norm import RMSNorm


def norm_comes_apart(producer, norm, consumer, rows: int) -> bool:
    """Whether ``norm`` between ``producer`` and ``consumer`` can be taken apart for this many rows: the
    producer adds its output into the residual itself and hands on half-normed rows, the consumer finishes."""
    give = getattr(producer, "adds_into_residual", None)
    take = getattr(consumer, "takes_half_normed", None)
    return (isinstance(norm, RMSNorm) and norm.weight is not None and give is not None and take is not None
            and give(rows) and take(rows))


@BLOCKS.register("prenorm_residual")
class PreNormResidual(Block):
    """``x += mixer(norm1(x)); x += ffn(norm2(x))``.

    Each add is done inside the norm that follows it, and the feed-forward's output stays pending
    until the next layer's (or the model's final) norm picks it up, as the reference defers its MLP
    residual (models/qwen3/src/model.rs:700-743,772-813).  The stream itself stays 32-bit.

    Where the step asks for it (``ctx.split_norms``) and the parts on both sides of a norm can (few rows,
    bfloat16: decode steps), the norm has no kernel of its own: the part before it adds into the residual and
    leaves half-normed rows, the part behind it finishes them (``HalfNormed``).  That holds for the norm
    between mixer and feed-forward and for the first norm of the block that runs next.  Whether it pays
    depends on the sizes (two launches less against longer tails of the products), so it is an option of
    the engine (``EngineConfig.split_norms``)."""

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheBinding,
                next_block: Optional[Block] = None) -> None:
        rows = stream.x.shape[0]
        if stream.half is not None:
            if stream.half_norm is not self.mixer_norm:
                raise RuntimeError("half-normed rows were made for another norm than this block's first")
            h, stream.half, stream.half_norm = stream.half, None, None
        else:
            h = self.mixer_norm.forward(stream.x, delta=stream.pending)
            stream.pending = None
        split = bool(getattr(ctx, "split_norms", False))
        if split and norm_comes_apart(self.mixer, self.feed_forward_norm, self.feed_forward, rows):
            h = self.mixer.forward(h, ctx, cache, sink=(stream.x, self.feed_forward_norm))
        else:
            a = self.mixer.forward(h, ctx, cache)
            h = self.feed_forward_norm.forward(stream.x, delta=a)
        if split and next_block is not None and norm_comes_apart(self.feed_forward, next_block.mixer_norm, next_block.mixer, rows):
            stream.half = self.feed_forward.forward(h, ctx, sink=(stream.x, next_block.mixer_norm))
            stream.half_norm = next_block.mixer_norm
        else:
            stream.pending = self.feed_forward.forward(h, ctx)
