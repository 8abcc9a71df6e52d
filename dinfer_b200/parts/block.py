"""Arrangements of a layer's four parts around the residual stream."""
from __future__ import annotations

from .base import BLOCKS, Block, CacheBinding, ResidualStream, StepContext


@BLOCKS.register("prenorm_residual")
class PreNormResidual(Block):
    """``x += mixer(norm1(x)); x += ffn(norm2(x))``.

    Each add is done inside the norm that follows it, and the feed-forward's output stays pending
    until the next layer's (or the model's final) norm picks it up, as the reference defers its MLP
    residual (models/qwen3/src/model.rs:700-743,772-813).  The stream itself stays 32-bit."""

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheBinding) -> None:
        h = self.mixer_norm.forward(stream.x, delta=stream.pending)
        a = self.mixer.forward(h, ctx, cache)
        h = self.feed_forward_norm.forward(stream.x, delta=a)
        stream.pending = self.feed_forward.forward(h, ctx)
