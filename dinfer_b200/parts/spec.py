"""What a model is made of, as data.

A model is an embedding, a list of layers, the order in which they run, a final norm and a head.
A layer names an arrangement (block) and four parts: mixer, feed-forward and their norms; each
part is a ``PartSpec``: the kind (a key of a registry) and its sizes and constants.  Nothing
here knows an architecture: an architecture's ``build_spec`` function fills these in from its
typed configuration.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default=None):
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    prefix: str                 # prefix of the layer's tensor names, e.g. "model.layers.3."
    block: str                  # arrangement of the parts, a key of the block registry
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  Weights belong to the layer, the cache to the entry: a layer named
    twice runs with the same weights and a cache of its own each time.  ``cache_from`` names an
    earlier entry whose cache this run reads instead of keeping one (it then writes none)."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_tensor: str
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    lm_head_tensor: str
    tie_word_embeddings: bool
    eos_token_ids: Tuple[int, ...] = ()
    embedding_scale: float = 1.0        # the embedding rows are multiplied by this on their way into the residual stream
    logit_softcap: float = 0.0          # > 0: logits = cap * tanh(logits / cap)

    def check(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if self.logit_softcap < 0 or not self.embedding_scale == self.embedding_scale:
            raise ValueError("logit_softcap must not be negative and embedding_scale must be a number")
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_from is not None:
                if not (0 <= e.cache_from < i):
                    raise ValueError(f"schedule entry {i}: cache_from must name an earlier entry")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {i}: cache_from must name an entry that owns its cache")


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part takes from the weight file."""
    name: str
    shape: Tuple[int, ...]
    # "float": kept in bfloat16 (a tensor the file stores in 32-bit stays so; everything is
    # 32-bit in the float32 engine).  "int": an integer table, kept as int32.
    kind: str = "float"
    optional: bool = False
    # how the random-weights mode fills it: "normal" (N(0, std)) or "ones" (1 + U(-jitter, jitter))
    init: str = "normal"
