"""A request's life: waiting -> running -> (preempted -> waiting ...) -> finished
(crates/core/src/request.rs:9-51,63-159)."""
from __future__ import annotations

import enum
import secrets
from dataclasses import dataclass, field
from typing import Hashable, List, Optional

from ..sampling.params import SamplingParams, TokenLogprobs


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class FinishReason(enum.Enum):
    STOP = "stop"          # an eos or stop token
    LENGTH = "length"      # max_tokens or max_model_len
    ABORT = "abort"


@dataclass
class Request:
    req_id: Hashable
    prompt_ids: List[int]
    params: SamplingParams
    seed: int = 0
    output_ids: List[int] = field(default_factory=list)
    num_computed: int = 0              # tokens whose keys are in the cache (or scheduled to be)
    num_placeholders: int = 0          # output tokens sampled on the device that the host has not read yet
    status: RequestStatus = RequestStatus.WAITING
    finish_reason: Optional[FinishReason] = None
    num_preemptions: int = 0
    logprobs: List[TokenLogprobs] = field(default_factory=list)   # one per output token, if asked for
    prompt_logprobs: List[Optional[TokenLogprobs]] = field(default_factory=list)   # one per prompt token (None first)
    # host clock (time.perf_counter): when the request came in, when the host read its first and its latest token
    t_arrival: float = 0.0
    t_first_token: float = 0.0
    t_last_token: float = 0.0

    def __post_init__(self):
        if self.params.seed is not None:
            self.seed = int(self.params.seed)
        elif self.seed == 0:
            self.seed = secrets.randbits(63)      # drawn once per request (crates/core/src/runner.rs:602)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    def token(self, i: int) -> int:
        n = len(self.prompt_ids)
        return self.prompt_ids[i] if i < n else self.output_ids[i - n]

    def tokens(self, lo: int, hi: int) -> List[int]:
        n = len(self.prompt_ids)
        if hi <= n:
            return self.prompt_ids[lo:hi]
        if lo >= n:
            return self.output_ids[lo - n:hi - n]
        return self.prompt_ids[lo:] + self.output_ids[:hi - n]

    @property
    def finished(self) -> bool:
        return self.status == RequestStatus.FINISHED
