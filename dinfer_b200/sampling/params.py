"""Per-request sampling options: names, defaults and ranges of the reference's ``SamplingParams``
(crates/core/src/sample.rs:81-205), without the text-level options (stop strings, logprobs,
grammars) that belong to the server."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    max_tokens: int = 256
    min_tokens: int = 0                 # eos / stop ids count only after this many tokens
    temperature: float = 1.0            # <= 1e-5 is greedy
    top_p: float = 1.0
    top_k: int = -1                     # -1 = off
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    seed: Optional[int] = None          # None: drawn once per request
    stop_token_ids: List[int] = field(default_factory=list)
    ignore_eos: bool = False

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 1e-5

    @property
    def has_penalties(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0
                or self.presence_penalty != 0.0)

    def validate(self) -> None:
        if self.temperature < 0.0:
            raise ValueError(f"temperature must be non-negative, got {self.temperature}")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < -1 or self.top_k == 0:
            raise ValueError(f"top_k must be -1 (disable) or at least 1, got {self.top_k}")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if not (0.0 < self.repetition_penalty <= 2.0):
            raise ValueError(f"repetition_penalty must be in (0, 2], got {self.repetition_penalty}")
        if not (-2.0 <= self.frequency_penalty <= 2.0):
            raise ValueError(f"frequency_penalty must be in [-2, 2], got {self.frequency_penalty}")
        if not (-2.0 <= self.presence_penalty <= 2.0):
            raise ValueError(f"presence_penalty must be in [-2, 2], got {self.presence_penalty}")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.min_tokens > self.max_tokens:
            raise ValueError(f"min_tokens {self.min_tokens} > max_tokens {self.max_tokens}")
