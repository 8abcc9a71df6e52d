"""The Python entry point: token ids in, token ids out.

    from dinfer_b200 import LLM, SamplingParams
    llm = LLM("/path/to/model", dtype="bfloat16", max_model_len=4096)
    outs = llm.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0, max_tokens=16))
    outs[0].output_ids

The options carry the names of the reference's ``dinfer serve`` flags / ``ServeOptions``
(bins/dinfer/src/main.rs:30-131, models/qwen3/src/service.rs:43-140).  The reference itself has no
in-process API (its only entry is the HTTP server); the loop below is its engine loop
(crates/core/src/engine.rs:538-728) without the thread and the channels: schedule -> step ->
sample -> update, until every request has finished.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Hashable, List, Optional, Sequence, Union


from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.loader import WeightSource
from .batch import StepEntry
from .request import Request
from .runner import ModelRunner
from .scheduler import Scheduler


@dataclass
class RequestOutput:
    req_id: Hashable
    prompt_ids: List[int]
    output_ids: List[int]
    finish_reason: str
    num_preemptions: int = 0


@dataclass
class EngineStats:
    steps: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    prefix_hit_tokens: int = 0        # prompt tokens found in the prefix cache (not run again)


class LLM:
    def __init__(self, model: Optional[str] = None, *, config: Optional[Dict[str, Any]] = None,
                 weights: Optional[WeightSource] = None, dtype: str = "bfloat16", max_model_len: int = 4096,
                 max_num_seqs: int = 16, max_num_batched_tokens: int = 2048, num_blocks: Optional[int] = None,
                 block_size: int = 16, gpu_memory_utilization: float = 0.9,
                 decode_exempt_from_budget: bool = True, long_prefill_token_threshold: int = 0,
                 enable_cuda_graph: bool = True, enable_prefix_caching: bool = False,
                 split_norms: bool = False, device: int = 0):
        """``model``: a folder with config.json and *.safetensors; or ``config`` (the config.json
        dictionary) with ``weights`` (any WeightSource, e.g. ``RandomSource``)."""
        self.engine_config = EngineConfig(
            max_model_len=max_model_len, max_num_seqs=max_num_seqs,
            max_num_batched_tokens=max_num_batched_tokens, num_blocks=num_blocks, block_size=block_size,
            gpu_memory_utilization=gpu_memory_utilization,
            decode_exempt_from_budget=decode_exempt_from_budget,
            long_prefill_token_threshold=long_prefill_token_threshold,
            enable_cuda_graph=enable_cuda_graph, enable_prefix_caching=enable_prefix_caching,
            split_norms=split_norms, dtype=dtype,
            device=device)
        if model is not None:
            self.runner = ModelRunner.from_dir(model, self.engine_config)
        elif config is not None and weights is not None:
            self.runner = ModelRunner(config, weights, self.engine_config)
        else:
            raise ValueError("give a model folder, or config and weights")
        self.scheduler = Scheduler(self.engine_config, self.runner.manager, self.runner.spec.eos_token_ids)
        self.sampler = Sampler(self.runner.device)
        self.stats = EngineStats()
        self._next_id = 0
        self._requests: Dict[Hashable, Request] = {}

    # ---- requests
    def add_request(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None,
                    req_id: Optional[Hashable] = None) -> Hashable:
        if req_id is None:
            req_id = self._next_id
            self._next_id += 1
        if req_id in self._requests:
            raise ValueError(f"request id {req_id!r} is in use")
        vocab = self.runner.spec.vocab_size
        if any((t < 0 or t >= vocab) for t in prompt_ids):
            raise ValueError(f"request {req_id!r}: a token id is outside the vocabulary [0, {vocab})")
        req = Request(req_id, list(prompt_ids), params or SamplingParams())
        self.scheduler.add_request(req)
        self._requests[req_id] = req
        return req_id

    def abort(self, req_id: Hashable) -> None:
        self.scheduler.abort(req_id)
        self._requests.pop(req_id, None)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # ---- one engine step
    def step(self) -> List[RequestOutput]:
        """Schedule, run, sample, update.  Returns the requests that finished in this step."""
        plan = self.scheduler.schedule()
        self._last_scheduled = len(plan.scheduled)
        finished = list(plan.finished)
        if plan.scheduled:
            entries, samplers = [], []
            for s in plan.scheduled:
                r = s.request
                entries.append(StepEntry(r.req_id, r.tokens(s.start, s.start + s.num_tokens),
                                         [s.num_tokens - 1] if s.samples else []))
                if s.samples:
                    samplers.append(r)
                self.stats.prompt_tokens += max(0, min(s.start + s.num_tokens, len(r.prompt_ids)) - s.start)
            logits = self.runner.step(entries)
            sampled: Dict[Hashable, int] = {}
            if samplers:
                toks = self.sampler(
                    logits, [r.params for r in samplers], [r.seed for r in samplers],
                    [len(r.output_ids) for r in samplers],
                    [(r.prompt_ids, r.output_ids) for r in samplers])
                host = toks.cpu().tolist()                   # the step's one device->host read
                sampled = {r.req_id: t for r, t in zip(samplers, host)}
                self.stats.generated_tokens += len(host)
            finished += self.scheduler.update(plan, sampled)
            self.stats.steps += 1
            if self.stats.steps % 256 == 0:
                self.runner.check_device_status()
        self.stats.preemptions = self.scheduler.num_preemptions
        self.stats.prefix_hit_tokens = self.runner.manager.prefix_hits
        outs = []
        for r in finished:
            self._requests.pop(r.req_id, None)
            outs.append(RequestOutput(r.req_id, r.prompt_ids, r.output_ids,
                                      r.finish_reason.value if r.finish_reason else "abort",
                                      r.num_preemptions))
        return outs

    # ---- whole generation
    def generate(self, prompt_token_ids: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[RequestOutput]:
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            params = [sampling_params or SamplingParams()] * len(prompt_token_ids)
        else:
            params = list(sampling_params)
            if len(params) != len(prompt_token_ids):
                raise ValueError("one SamplingParams per prompt")
        import copy
        ids = [self.add_request(p, copy.copy(sp)) for p, sp in zip(prompt_token_ids, params)]
        done: Dict[Hashable, RequestOutput] = {}
        idle = 0
        while self.has_unfinished():
            outs = self.step()
            for o in outs:
                done[o.req_id] = o
            idle = idle + 1 if (not outs and self._last_scheduled == 0) else 0
            if idle > 100:
                raise RuntimeError("the scheduler makes no progress")
        self.runner.check_device_status()
        return [done[i] for i in ids]
