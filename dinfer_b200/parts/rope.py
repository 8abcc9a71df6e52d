"""Rotary position encoding: pairs ``(i, i + rot/2)`` (neox) or ``(2i, 2i + 1)`` (interleaved), over the whole head
or its first ``rotary_dim`` elements, positions optionally divided by a factor (linear scaling).

A position encoding is a helper of a mixer.  Interface:
  ``fused_table()`` -> the ``[max_positions, rot]`` f32 table ``cos | sin`` when the rotation can be
                      done inside the q/k post-processing kernel, else None;
  ``apply(q, k, ctx)`` -> for encodings that are not a table rotation: change the ``[T, heads, D]``
                      views of q and k in place (called between the head norm and the cache write).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import POSITION_ENCODINGS, PositionEncoding

_TABLES: Dict[Tuple, torch.Tensor] = {}


def rope_table(rotary_dim: int, theta: float, max_positions: int, device, scaling_factor: float = 1.0) -> torch.Tensor:
    """``[p, i] = cos(p f_i)``, ``[p, rot/2 + i] = sin(p f_i)``, ``f_i = theta^(-2i/rot) / scaling_factor``: angles in
    64-bit, stored in 32-bit (crates/layers/src/nn.rs:157-173)."""
    key = (rotary_dim, float(theta), max_positions, str(device), float(scaling_factor))
    t = _TABLES.get(key)
    if t is None:
        half = rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        inv_freq = 1.0 / (float(theta) ** (2.0 * i / rotary_dim)) / float(scaling_factor)
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        t = torch.cat([ang.cos(), ang.sin()], dim=1).to(torch.float32).to(device).contiguous()
        _TABLES[key] = t
    return t


@POSITION_ENCODINGS.register("rope")
@POSITION_ENCODINGS.register("rope_neox")
class RotaryNeox(PositionEncoding):
    """params: ``head_dim``, ``theta``, ``max_positions``, optional ``rotary_dim`` (default: the whole head),
    ``style`` ("neox", the default: element i turns with i + rot/2; "interleaved": element 2i with 2i + 1) and
    ``scaling_factor`` (positions divided by it; default 1).  All of it is the table and one flag of the q/k kernel."""

    def __init__(self, params, env, prefix=""):
        super().__init__(params, env, prefix)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        style = params.get("style", "neox")
        if style not in ("neox", "interleaved"):
            raise ValueError(f"rotary style {style!r}: neox or interleaved")
        self.interleaved = style == "interleaved"
        self.scaling_factor = float(params.get("scaling_factor", 1.0))
        if not self.scaling_factor > 0:
            raise ValueError("scaling_factor must be positive")
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self._table: Optional[torch.Tensor] = None

    fused = True

    def fused_table(self) -> Optional[torch.Tensor]:
        if self._table is None:
            self._table = rope_table(self.rotary_dim, self.theta, self.max_positions, self.env.device,
                                     self.scaling_factor)
        return self._table

    def apply(self, q, k, ctx) -> None:       # the rotation is always fused
        raise NotImplementedError


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    fused = True

    def fused_table(self):
        return None

    def apply(self, q, k, ctx) -> None:
        return None
