"""The Python entry point: token ids in, token ids out.

    from dinfer_b200 import LLM, SamplingParams
    llm = LLM("/path/to/model", dtype="bfloat16", max_model_len=4096)
    outs = llm.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0, max_tokens=16))
    outs[0].output_ids

or step by step, for a caller that streams tokens on:

    rid = llm.add_request([1, 2, 3], SamplingParams(max_tokens=16))
    while llm.has_unfinished():
        finished = llm.step()                   # RequestOutput of every request that ended
        fresh = llm.take_new_tokens()           # {request: tokens it got since the last look}

The options carry the names of the reference's ``dinfer serve`` flags / ``ServeOptions``
(bins/dinfer/src/main.rs:30-131, models/qwen3/src/service.rs:43-140).  The reference itself has no
in-process API (its only entry is the HTTP server); the loop below is its engine loop
(crates/core/src/engine.rs:538-728) without the thread and the channels: schedule -> step ->
sample -> update, until every request has finished.  With ``async_scheduling`` (the default) one step
is kept in flight: step n + 1 is scheduled and launched while step n runs, its requests' newest tokens
taken on the device from step n's sampling, and only then are step n's tokens read and its requests
updated; ``step()`` then returns what finished one launch earlier.
"""
from __future__ import annotations

import copy
import time
from dataclasses import dataclass
from typing import Any, Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams, TokenLogprobs, generation_defaults
from ..sampling.sampler import Sampler
from ..weights.loader import WeightSource
from .batch import StepEntry
from .request import Request
from .runner import ModelRunner
from .scheduler import NativeScheduler, Scheduler


@dataclass
class RequestOutput:
    req_id: Hashable
    prompt_ids: List[int]
    output_ids: List[int]
    finish_reason: str
    num_preemptions: int = 0
    logprobs: Optional[List[TokenLogprobs]] = None      # one per output token, if the request asked for them
    prompt_logprobs: Optional[List[Optional[TokenLogprobs]]] = None   # one per prompt token, None for the first
    # seconds on the host's clock, as the reference's metrics define them (crates/server/src/metrics.rs:63-142):
    # from arrival to the first token, mean time per token after the first, from arrival to the end
    ttft_s: float = 0.0
    tpot_s: float = 0.0
    e2e_s: float = 0.0


@dataclass
class EngineStats:
    steps: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    prefix_hit_tokens: int = 0        # prompt tokens found in the prefix cache (not run again)
    # where the host's time of the steps went, in seconds (the reference prints such segments with HOST_TIME=1,
    # crates/core/src/engine.rs:664-711): deciding the step, building its plan and queueing its kernels, and waiting
    # for and applying the tokens of the step before (with one step in flight the wait is where the device shows)
    host_schedule_s: float = 0.0
    host_launch_s: float = 0.0
    host_collect_s: float = 0.0


class _InFlight:
    """A step whose device work is queued and whose tokens the host has not read."""

    def __init__(self, plan, samplers: List[Request], row: Dict[Hashable, int]):
        self.plan = plan
        self.samplers = samplers
        self.row = row                      # request -> its row in the step's sampled tokens
        self.host: Optional[torch.Tensor] = None
        self.event: Optional[torch.cuda.Event] = None
        self.logprobs = None                # (ids, logprobs, rank) on the device, if a row asked for them
        self.taken_ahead = set()            # requests whose token of this step the next step took on the device


class LLM:
    def __init__(self, model: Optional[str] = None, *, config: Optional[Dict[str, Any]] = None,
                 weights: Optional[WeightSource] = None, dtype: str = "bfloat16", max_model_len: int = 4096,
                 max_num_seqs: int = 16, max_num_batched_tokens: int = 2048, num_blocks: Optional[int] = None,
                 block_size: int = 16, gpu_memory_utilization: float = 0.9,
                 decode_exempt_from_budget: bool = True, long_prefill_token_threshold: int = 0,
                 enable_cuda_graph: bool = True, enable_prefix_caching: bool = False,
                 split_norms: Any = False, async_scheduling: bool = True, mixed_cuda_graph: bool = True,
                 allow_unused_tensors: bool = False, native_host: bool = True, device: int = 0):
        """``model``: a folder with config.json and *.safetensors; or ``config`` (the config.json
        dictionary) with ``weights`` (any WeightSource, e.g. ``RandomSource``)."""
        self.engine_config = EngineConfig(
            max_model_len=max_model_len, max_num_seqs=max_num_seqs,
            max_num_batched_tokens=max_num_batched_tokens, num_blocks=num_blocks, block_size=block_size,
            gpu_memory_utilization=gpu_memory_utilization,
            decode_exempt_from_budget=decode_exempt_from_budget,
            long_prefill_token_threshold=long_prefill_token_threshold,
            enable_cuda_graph=enable_cuda_graph, enable_prefix_caching=enable_prefix_caching,
            split_norms=split_norms, async_scheduling=async_scheduling, mixed_cuda_graph=mixed_cuda_graph,
            allow_unused_tensors=allow_unused_tensors, native_host=native_host, dtype=dtype,
            device=device)
        # what a request gets that brings no SamplingParams of its own: the model folder's generation_config.json
        # (temperature, top_p, top_k) over the built-in defaults
        self.default_sampling_params = generation_defaults(model)
        if model is not None:
            self.runner = ModelRunner.from_dir(model, self.engine_config)
        elif config is not None and weights is not None:
            self.runner = ModelRunner(config, weights, self.engine_config)
        else:
            raise ValueError("give a model folder, or config and weights")
        native = hasattr(self.runner.manager, "fill_decode_plan")      # the C++ cache manager takes the C++ scheduler
        self.scheduler = (NativeScheduler if native else Scheduler)(self.engine_config, self.runner.manager,
                                                                    self.runner.spec.eos_token_ids)
        self.sampler = Sampler(self.runner.device)
        self.stats = EngineStats()
        self._next_id = 0
        self._requests: Dict[Hashable, Request] = {}
        # scheduling ahead: the step in flight, and pinned buffers its tokens are copied to (two: one being
        # read by the host while the next step's copy is queued)
        self._ahead = bool(self.engine_config.async_scheduling)
        self._inflight: Optional[_InFlight] = None
        self._num_penalized = 0
        rows = self.runner.sampled.numel()
        self._tok_host = [torch.empty(rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._tok_turn = 0
        self._new_tokens: Dict[Hashable, List[int]] = {}   # tokens appended since take_new_tokens() was last called

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
        req = Request(req_id, list(prompt_ids), params or copy.copy(self.default_sampling_params))
        req.t_arrival = time.perf_counter()
        if any(t >= vocab for t in req.params.logit_bias):
            raise ValueError(f"request {req_id!r}: a logit_bias token id is outside the vocabulary [0, {vocab})")
        self.scheduler.add_request(req)
        self._requests[req_id] = req
        self._num_penalized += int(req.params.needs_host_history)
        return req_id

    def abort(self, req_id: Hashable) -> None:
        self.scheduler.abort(req_id)
        self._forget(req_id)

    def _forget(self, req_id: Hashable) -> None:
        req = self._requests.pop(req_id, None)
        if req is not None:
            self._num_penalized -= int(req.params.needs_host_history)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None

    # ---- one engine step
    def step(self) -> List[RequestOutput]:
        """Schedule, run, sample, update.  Returns the requests known to have finished: those of this step,
        or, when scheduling ahead, those of the step launched by the call before."""
        # penalties need every earlier token on the host, log-probabilities are read with the tokens: such steps
        # run one at a time
        ahead = self._ahead and self._num_penalized == 0
        finished: List[Request] = []
        if not ahead and self._inflight is not None:
            finished += self._collect()
        t0 = time.perf_counter()
        plan = self.scheduler.schedule(lookahead=ahead)
        self._last_scheduled = len(plan.scheduled)
        finished += plan.finished
        t1 = time.perf_counter()
        launched = self._launch(plan) if plan.scheduled else None
        t2 = time.perf_counter()
        if self._inflight is not None:              # the step before this one: its tokens have arrived by now
            finished += self._collect()
        self._inflight = launched
        if launched is not None and not ahead:
            finished += self._collect()
        t3 = time.perf_counter()
        self.stats.host_schedule_s += t1 - t0
        self.stats.host_launch_s += t2 - t1
        self.stats.host_collect_s += t3 - t2
        self.stats.preemptions = self.scheduler.num_preemptions
        self.stats.prefix_hit_tokens = self.runner.manager.prefix_hits
        outs = []
        for r in finished:
            self._forget(r.req_id)
            n = len(r.output_ids)
            outs.append(RequestOutput(r.req_id, r.prompt_ids, r.output_ids,
                                      r.finish_reason.value if r.finish_reason else "abort",
                                      r.num_preemptions,
                                      r.logprobs if r.params.logprobs is not None else None,
                                      r.prompt_logprobs if r.params.prompt_logprobs is not None else None,
                                      ttft_s=max(0.0, r.t_first_token - r.t_arrival) if n else 0.0,
                                      tpot_s=(r.t_last_token - r.t_first_token) / (n - 1) if n > 1 else 0.0,
                                      e2e_s=max(0.0, r.t_last_token - r.t_arrival) if n else 0.0))
        return outs

    def _launch(self, plan) -> "_InFlight":
        """Queue the step's device work and the copy of its sampled tokens to the host; wait for nothing."""
        prev_row = self._inflight.row if self._inflight is not None else {}
        entries, samplers, generated, scored = [], [], [], []
        for s in plan.scheduled:
            r = s.request
            end = s.start + s.num_tokens
            if end > r.num_tokens:                  # its newest token is still on the device: named by its row
                toks = r.tokens(s.start, r.num_tokens) + [-(prev_row[r.req_id] + 1)]
                self._inflight.taken_ahead.add(r.req_id)
            else:
                toks = r.tokens(s.start, end)
            want = [s.num_tokens - 1] if s.samples else []
            if r.params.prompt_logprobs is not None and s.start == 0:
                r.prompt_logprobs = [None]          # (a request that was preempted is scored again from the start)
            if r.params.prompt_logprobs is not None and s.start < len(r.prompt_ids) - 1:
                # every position of this portion that is followed by another prompt token: its logits say how
                # likely that token was
                if len(r.prompt_logprobs) == s.start + 1:
                    upto = min(end, len(r.prompt_ids) - 1)
                    scored.append((r, len(entries), s.start, upto))
                    want = list(range(upto - s.start)) + want
            entries.append(StepEntry(r.req_id, toks, want))
            if s.samples:
                samplers.append(r)
                generated.append(s.num_generated)
            self.stats.prompt_tokens += max(0, min(end, len(r.prompt_ids)) - s.start)
        logits = self.runner.step(entries, placeholders=True)
        if scored:                                  # rows come in the order of the entries and of their wanted places
            logits = self._score_prompts(logits, entries, scored)
        flight = _InFlight(plan, samplers, {r.req_id: i for i, r in enumerate(samplers)})
        if samplers:
            out = self.runner.sampled[:len(samplers)]
            self.sampler(logits, [r.params for r in samplers], [r.seed for r in samplers], generated,
                         [(r.prompt_ids, r.output_ids) for r in samplers], out=out)
            k = self._tok_turn
            self._tok_turn = 1 - k
            flight.host = self._tok_host[k]
            flight.host[:len(samplers)].copy_(out, non_blocking=True)     # the step's one device->host read
            flight.event = torch.cuda.Event()
            flight.event.record()
            flight.logprobs = self.sampler.last_logprobs
        self.stats.steps += 1
        if self.stats.steps % 256 == 0:
            self.runner.check_device_status()
        return flight

    def _score_prompts(self, logits: torch.Tensor, entries, scored) -> torch.Tensor:
        """Log-probabilities of the prompt tokens from the rows asked for them; returns the rows that are sampled
        from.  (Such requests run one step at a time, so reading the result here stalls nothing that matters.)"""
        from ..sampling.sampler import logprobs as row_logprobs
        first_row, n = [], 0
        for e in entries:
            first_row.append(n)
            n += len(e.want)
        keep = torch.ones(n, dtype=torch.bool, device=logits.device)
        for r, ei, lo, hi in scored:
            a = first_row[ei]
            rows = logits[a:a + hi - lo]
            targets = torch.tensor(r.prompt_ids[lo + 1:hi + 1], dtype=torch.int32, device=logits.device)
            k = r.params.prompt_logprobs
            ids, lps, rank = (t.cpu().tolist() for t in row_logprobs(rows, targets, k))
            for i in range(hi - lo):
                r.prompt_logprobs.append(TokenLogprobs(ids[i][0], lps[i][0], rank[i], ids[i][1:1 + k], lps[i][1:1 + k]))
            keep[a:a + hi - lo] = False
        return logits[keep]

    def _collect(self) -> List[Request]:
        """Wait for the tokens of the step in flight and update its requests."""
        flight, self._inflight = self._inflight, None
        sampled: Dict[Hashable, int] = {}
        if flight.samplers:
            flight.event.synchronize()
            host = flight.host[:len(flight.samplers)].tolist()
            sampled = {r.req_id: t for r, t in zip(flight.samplers, host)}
            # what a step ahead computed for a request that has finished meanwhile is dropped, not counted
            self.stats.generated_tokens += sum(1 for r in flight.samplers if not r.finished)
        before = {r.req_id: len(r.output_ids) for r in flight.samplers}
        done = self.scheduler.update(flight.plan, sampled)
        now = time.perf_counter()
        for r in flight.samplers:                   # what was appended (a dropped token is not)
            if len(r.output_ids) > before[r.req_id]:
                self._new_tokens.setdefault(r.req_id, []).extend(r.output_ids[before[r.req_id]:])
                if before[r.req_id] == 0 and r.t_first_token == 0.0:
                    r.t_first_token = now
                r.t_last_token = now
        manager = self.runner.manager
        if manager.prefix_caching:                  # tokens the next step took on the device: the cache learns them
            for rid in flight.taken_ahead:
                if rid in manager:
                    manager.resolve(rid, [sampled[rid]])
        if flight.logprobs is not None:
            ids, lps, rank = (t.cpu().tolist() for t in flight.logprobs)
            for i, r in enumerate(flight.samplers):
                k = r.params.logprobs
                if k is not None and r.output_ids and r.output_ids[-1] == ids[i][0]:
                    r.logprobs.append(TokenLogprobs(ids[i][0], lps[i][0], rank[i], ids[i][1:1 + k], lps[i][1:1 + k]))
        return done

    def take_new_tokens(self) -> Dict[Hashable, List[int]]:
        """The tokens every request has got since the last call, in order (for a caller that streams them on):
        ``while llm.has_unfinished(): done = llm.step(); fresh = llm.take_new_tokens()``."""
        fresh, self._new_tokens = self._new_tokens, {}
        return fresh

    # ---- whole generation
    def generate(self, prompt_token_ids: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[RequestOutput]:
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            params = [sampling_params or self.default_sampling_params] * len(prompt_token_ids)
        else:
            params = list(sampling_params)
            if len(params) != len(prompt_token_ids):
                raise ValueError("one SamplingParams per prompt")
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
