"""Interfaces of the parts and the registries that map a ``PartSpec.kind`` to its class.

A part is built from ``(spec.params, env)``, declares the tensors it takes, receives them in
``bind`` and then only sees activations, the step's ``StepContext`` and (a mixer) its cache.
No part knows which model it is in.

    Mixer           forward(x [T, h], ctx, cache) -> [T, h];  cache_need() says what it keeps
    FeedForward     forward(x [T, h], ctx) -> [T, h]
    Norm            forward(residual f32 [T, h], delta | None, rows | None) -> normed [R, h]
    PositionEncoding  a mixer's helper; see parts/rope.py
    Block           forward(stream: ResidualStream, ctx, cache) -> None   (arranges the four)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from .spec import PartSpec, TensorDecl


# ---------------------------------------------------------------- what a mixer keeps

@dataclass(frozen=True)
class KvCacheNeed:
    """Keys and values of every token (``window`` None) or of the last ``window`` tokens, in pages of
    ``block_size`` tokens (None: the engine's page size)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    block_size: Optional[int] = None

    def group_key(self):
        # layers whose pages live and die together: same span of tokens, same page size
        return ("kv", self.window, self.block_size)


@dataclass(frozen=True)
class StateNeed:
    """A per-request state of fixed size (``shape`` elements of ``dtype``), zeroed for a new request."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ---------------------------------------------------------------- what a part sees of a step

@dataclass
class CacheGroupView:
    """One cache group's view of the step: pages of the requests and the slot of each new token."""
    block_size: int
    block_table: torch.Tensor          # [B, max_blocks] int32, -1 where no page is held
    slot_mapping: torch.Tensor         # [T] int32, block*block_size + offset (-1: not stored)
    window: Optional[int] = None


@dataclass
class StepContext:
    """The batch of one step, on the device (and the few numbers the host needs to launch)."""
    num_tokens: int
    num_reqs: int
    positions: torch.Tensor            # [T] int32, absolute position of each token
    cu_seqlens: torch.Tensor           # [B+1] int32, offsets of the requests' tokens
    seq_lens: torch.Tensor             # [B] int32, length of each request after this step
    groups: List[CacheGroupView]
    state_slots: torch.Tensor          # [B] int32, slot of each request's fixed-size state
    state_fresh: torch.Tensor          # [B] int32, 1 where the request starts (state must be zeroed)
    max_q_len: int                     # longest portion in the batch
    max_seq_len: int                   # longest request after the step
    all_decode: bool                   # every request brings exactly one token
    any_decode: bool = True            # some request brings exactly one token
    any_prefill: bool = True           # some request brings more than one
    decode_splits: int = 0             # > 0: the decode attention uses this many key splits (CUDA graphs)
    max_prefill_seq_len: int = 0       # longest request among those that bring more than one token (0: not known,
                                       # take max_seq_len); inside a captured graph a bound for all its replays
    split_norms: bool = False          # norms between two products may be taken apart (see HalfNormed)
    prev_tokens: Optional[torch.Tensor] = None   # int32 [rows]: a token id -(r + 1) stands for prev_tokens[r]
    # host copies for parts written in plain torch (tests, toy parts)
    cu_seqlens_host: Sequence[int] = ()
    seq_lens_host: Sequence[int] = ()
    state_slots_host: Sequence[int] = ()
    state_fresh_host: Sequence[int] = ()
    # numbers a part derives from the host copies once per step and shares between its layers
    derived: Dict[Any, Any] = field(default_factory=dict)


@dataclass
class CacheBinding:
    """The cache a mixer works on in one schedule entry."""
    kv: Optional[torch.Tensor] = None      # [num_blocks, 2, Hkv, block_size, D] of this entry
    group: int = -1                        # index into StepContext.groups
    write: bool = True                     # False when the entry reads another entry's cache
    state: Optional[torch.Tensor] = None   # [num_slots, *shape] of this entry


@dataclass
class BuildEnv:
    """What a part needs to know about the engine it is built into."""
    device: torch.device
    act_dtype: torch.dtype             # torch.bfloat16 or torch.float32
    hidden_size: int
    max_positions: int


# ---------------------------------------------------------------- base classes

class Part:
    def __init__(self, params: Mapping[str, Any], env: BuildEnv, prefix: str = ""):
        self.params = dict(params)
        self.env = env
        self.prefix = prefix

    def declare(self) -> List[TensorDecl]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def kernel_libraries(self) -> List[str]:
        """Names of the kernel libraries the part launches (built before the first step)."""
        return []


@dataclass
class HalfNormed:
    """Rows on their way through an RMSNorm that is taken apart between two matrix products: ``xw`` is the
    32-bit residual times the norm's weight, rounded to the activation type, and ``sums[p, t]`` are partial
    sums of the squares of residual row t.  What is missing is the division by the row's root mean square,
    ``rsqrt(sum_p sums[p, t] / size + eps)``; it commutes with a matrix product, so the product that
    consumes the rows applies it to its result."""
    xw: torch.Tensor
    sums: torch.Tensor
    parts: int
    size: int
    eps: float

    @property
    def shape(self):
        return self.xw.shape


class Mixer(Part):
    """Optional beside ``forward``, for parts whose first and last operation can take an RMSNorm apart (see
    ``HalfNormed``): ``takes_half_normed(rows) -> bool`` says that ``forward`` accepts a ``HalfNormed`` as
    ``x`` for this many rows; ``adds_into_residual(rows) -> bool`` says that ``forward(..., sink=(residual,
    norm))`` adds the part's output into the residual itself and returns the ``HalfNormed`` input of the
    next part instead of the output.  A part without them always gets and gives plain tensors."""

    # A mixer with per-request state says here whether its forward can be captured in a CUDA graph: it must read the
    # step's state slots and fresh flags from the device tensors of the context (``ctx.state_slots``,
    # ``ctx.state_fresh``, ``ctx.cu_seqlens``), never from their host copies, and take rows without a request (the
    # padding of a captured batch) in its stride: those carry the spare slot ``cache.state.shape[0] - 1``, which no
    # request ever holds.  Mixers without state are always capturable.
    graph_capturable = False

    def cache_need(self):
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """The optional ``takes_half_normed`` / ``adds_into_residual`` of a ``Mixer`` hold here too."""

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    # True: the q/k post-processing kernel does the whole encoding (a table rotation or nothing);
    # False: the mixer calls apply(q, k, ctx) between the head norm and the cache write.
    fused = False

    def fused_table(self) -> Optional[torch.Tensor]:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx: "StepContext") -> None:
        raise NotImplementedError


@dataclass
class ResidualStream:
    """The 32-bit residual ``x`` and either a part's output that has not been added to it yet (``pending``) or
    the input of the next block's mixer, already added and half normed by the part before (``half``, made for
    the norm ``half_norm``)."""
    x: torch.Tensor
    pending: Optional[torch.Tensor] = None
    half: Optional["HalfNormed"] = None
    half_norm: Optional["Norm"] = None


class Block:
    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward, feed_forward_norm: Norm):
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm

    def parts(self) -> List[Part]:
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheBinding,
                next_block: Optional["Block"] = None) -> None:
        """``next_block``: the block that runs after this one (None after the last), for arrangements that
        hand their output to its first norm in another form than a pending tensor."""
        raise NotImplementedError


# ---------------------------------------------------------------- registries

class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Any] = {}

    def register(self, kind: str, cls=None, *, replace: bool = False):
        def put(c):
            if kind in self._items and not replace:
                raise ValueError(f"{self.what} {kind!r} is already registered")
            self._items[kind] = c
            return c
        return put if cls is None else put(cls)

    def unregister(self, kind: str) -> None:
        self._items.pop(kind, None)

    def get(self, kind: str):
        if kind not in self._items:
            raise KeyError(f"unknown {self.what} {kind!r} (registered: {', '.join(sorted(self._items))})")
        return self._items[kind]

    def kinds(self):
        return sorted(self._items)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")


def build_part(registry: Registry, spec: PartSpec, env: BuildEnv, prefix: str) -> Part:
    return registry.get(spec.kind)(spec.params, env, prefix)
