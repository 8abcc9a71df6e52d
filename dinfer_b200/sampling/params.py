"""Per-request sampling options: names, defaults and ranges of the reference's ``SamplingParams``
(crates/core/src/sample.rs:81-205), without the options that need the tokenizer or the server (stop strings,
grammars)."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional


MAX_LOGPROBS = 32          # the most candidates a token's log-probabilities list (crates/kernels/cuda/sampling.cu:382)
MAX_LOGIT_BIAS = 300       # crates/core/src/sample.rs:104


@dataclass
class TokenLogprobs:
    """Log-probabilities at one generated token."""
    token_id: int
    logprob: float
    rank: int                           # tokens strictly more likely than this one
    top_ids: List[int] = field(default_factory=list)
    top_logprobs: List[float] = field(default_factory=list)


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
    # None: no log-probabilities; k >= 0: every generated token comes with its log-probability and rank under
    # log_softmax of the model's logits (before bias, penalties and temperature) and with the k most likely tokens
    logprobs: Optional[int] = None
    # k >= 0: every prompt position but the first comes with the log-probability and rank of its token given the
    # tokens before it, and with the k most likely tokens there (the prompt is then run whole, not taken from the
    # prefix cache)
    prompt_logprobs: Optional[int] = None
    # token id -> bias added to the logits before the penalties (at most 300 entries)
    logit_bias: Dict[int, float] = field(default_factory=dict)

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 1e-5

    @property
    def has_penalties(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0
                or self.presence_penalty != 0.0)

    @property
    def needs_host_history(self) -> bool:
        """Options whose step cannot be launched before the last step's tokens are on the host."""
        return self.has_penalties or self.logprobs is not None or self.prompt_logprobs is not None

    def validate(self) -> None:
        if self.logprobs is not None and not (0 <= self.logprobs <= MAX_LOGPROBS):
            raise ValueError(f"logprobs must be in [0, {MAX_LOGPROBS}], got {self.logprobs}")
        if self.prompt_logprobs is not None and not (0 <= self.prompt_logprobs <= MAX_LOGPROBS):
            raise ValueError(f"prompt_logprobs must be in [0, {MAX_LOGPROBS}], got {self.prompt_logprobs}")
        if len(self.logit_bias) > MAX_LOGIT_BIAS:
            raise ValueError(f"logit_bias takes at most {MAX_LOGIT_BIAS} entries, got {len(self.logit_bias)}")
        for t, b in self.logit_bias.items():
            if isinstance(t, bool) or not isinstance(t, int) or t < 0:
                raise ValueError(f"logit_bias: {t!r} is not a token id")
            if not (-100.0 <= float(b) <= 100.0):
                raise ValueError(f"logit_bias: bias {b} of token {t} is outside [-100, 100]")
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


def generation_defaults(model_dir: Optional[str]) -> SamplingParams:
    """The sampling defaults a model folder brings: temperature, top_p and top_k of its ``generation_config.json``
    over the built-in defaults, as the reference's server takes them (models/qwen3/src/service.rs:477-493).  A
    folder without the file, or no folder, gives the built-in defaults."""
    sp = SamplingParams()
    path = os.path.join(model_dir, "generation_config.json") if model_dir else None
    if path and os.path.isfile(path):
        try:
            with open(path, "r", encoding="utf-8") as f:
                g = json.load(f)
        except (OSError, json.JSONDecodeError):
            return sp
        if isinstance(g, dict):
            t, p, k = g.get("temperature"), g.get("top_p"), g.get("top_k")
            if isinstance(t, (int, float)) and not isinstance(t, bool):
                sp.temperature = float(t)
            if isinstance(p, (int, float)) and not isinstance(p, bool):
                sp.top_p = float(p)
            if isinstance(k, int) and not isinstance(k, bool):
                sp.top_k = int(k) if k > 0 else -1
    return sp
