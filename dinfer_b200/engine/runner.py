"""The step function.

``ModelRunner.step(entries)`` takes a batch of (request, its next tokens, wanted places): portions of
prompts beside single decoded tokens, cut anywhere.  It allocates pages for the new tokens, runs
only those tokens as one batch against the cache that earlier steps left, and returns the f32 logits
at the wanted places ``[R, V]`` (device tensor, in the order of the entries and of their ``want``).
Generation (scheduler + sampling) and trace replay both drive this one function.

It stands where the reference has ``Runner::execute`` -> ``Qwen3Executor::forward_sample`` ->
``Qwen3Model::forward`` (crates/core/src/runner.rs:362-429, models/qwen3/src/executor.rs:977-1026,
models/qwen3/src/model.rs:684-832), with sampling kept out of it.

How a step reaches the device is an optimisation, never a difference in meaning: decode-only steps replay a
CUDA graph per batch bucket, steps with prompt portions replay one where their shape comes again
(``graph_shape``), every other step launches its kernels one by one.
"""
from __future__ import annotations

import dataclasses
import math
import time
from typing import Any, Dict, Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager, GroupSpec
from ..config.engine_config import EngineConfig
from ..config.model_config import read_config_json
from ..config.registry import resolve_architecture
from ..kernels import lib as kernel_lib
from ..models.decoder import DecoderModel
from ..parts.base import BuildEnv, CacheBinding, KvCacheNeed, StateNeed
from ..weights.loader import SafetensorsSource, WeightSource, load_tensors
from .batch import DecodePlan, OutOfPages, PlanBuilder, StepEntry

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def graph_shape(prompt_lens: Sequence[int], num_decodes: int, budget: int, buckets: Sequence[int],
                place_counts: Sequence[int], small_max: int, padded_limit: int, longest: Optional[int] = None):
    """The shape of the captured graph a step with prompt portions replays, as (prompt tokens after padding,
    prompt places, decode bucket), or None for a step that runs kernel by kernel.  ``prompt_lens``: the tokens of
    the step's prompt portions; ``place_counts``: the numbers of prompt places graphs are made with, rising (the
    padding takes a place too; a place without tokens still counts one row-tile pair per head in the bound the
    attention kernel's grid is made from, hence more than one size); ``small_max``: up to so many prompt tokens are padded to a power of two
    (from 16); ``padded_limit``: up to so many are padded to a multiple of 128 (256 beyond 1024); portions that
    fill ``budget`` exactly need no padding.  ``longest``: the most tokens one place may hold (the longest request
    the cache tables and the position table are made for); a step whose dummy portion, or whose capture (dummy
    portions only), would need a longer one runs kernel by kernel."""
    have = sum(prompt_lens)
    if not prompt_lens or any(n < 2 for n in prompt_lens):
        return None
    if have == budget:
        total = budget
    elif have <= min(small_max, budget):
        total = 16
        while total < have:
            total *= 2
    else:
        unit = 128 if have <= 1024 else 256
        total = min(budget, (have + unit - 1) // unit * unit)
        if total > padded_limit:
            return None
    if total > budget:
        return None                                          # no room for the dummy portion
    need = len(prompt_lens) + (1 if total > have else 0)
    places = next((p for p in place_counts if p >= need), None)
    bucket = 0 if not num_decodes else next((b for b in buckets if b >= num_decodes), None)
    if places is None or bucket is None:
        return None
    if longest is not None and (total - have > longest or capture_places(total, places, bucket, longest) is None):
        return None
    return total, places, bucket


def capture_places(total: int, n_places: int, bucket: int, longest: int):
    """The dummy batch a graph of this shape is captured on, as (-1, tokens) per place: ``total`` prompt tokens
    spread over the prompt places, none longer than ``longest``, then the bucket's one-token places.  None when
    the places cannot hold them."""
    places, rest = [], total
    for _ in range(n_places):
        n = min(rest, longest)
        places.append((-1, n))
        rest -= n
    if rest > 0:
        return None
    return places + [(-1, 1)] * bucket


class ModelRunner:
    # the numbers of prompt places captured mixed steps are made with, and the most prompt tokens of a step that is
    # padded up to a power of two to replay a graph (see graph_shape)
    PROMPT_PLACES = (4, 16)
    PADDED_PROMPT_TOKENS = 128
    # mixed steps whose prompt requests all stay within this many tokens replay graphs of their own, captured with
    # that bound in the step context, so that a part may choose its kernel for short contexts there
    SHORT_CONTEXT = 512

    def __init__(self, config_dict: Dict[str, Any], source: WeightSource, engine: EngineConfig):
        engine.check()
        if not torch.cuda.is_available():
            raise RuntimeError("dinfer_b200 runs on a CUDA device (sm_100a); none is visible and there "
                               "is no CPU path")
        self.engine = engine
        self.device = torch.device("cuda", engine.device)
        torch.cuda.set_device(self.device)
        # true 32-bit means no reduced-precision matrix mode anywhere, library calls included
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        # the library's bfloat16 products fold their K splits in 32-bit, like the engine's own kernels do, so that
        # the same tokens run in a large step and in a small one differ by one rounding only
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self.act_dtype = _TORCH_DTYPE[engine.dtype]
        arch = resolve_architecture(config_dict)
        self.config = arch.parse_config(config_dict)
        self.spec = arch.build_spec(self.config)
        if engine.max_model_len > self.spec.max_positions:
            raise ValueError(f"max_model_len {engine.max_model_len} exceeds the model's "
                             f"max_position_embeddings {self.spec.max_positions}")
        env = BuildEnv(self.device, self.act_dtype, self.spec.hidden_size, self.spec.max_positions)
        self.model = DecoderModel(self.spec, env)
        # where the start-up time goes, in seconds (the reference logs such phases: crates/layers/src/load.rs:35-136)
        t0 = time.perf_counter()
        self.unused_tensors: List[str] = []
        tensors = load_tensors(source, self.model.declarations(), self.act_dtype, self.device,
                               allow_unexpected=engine.allow_unused_tensors, unused=self.unused_tensors)
        if self.unused_tensors:
            import sys
            print(f"[dinfer_b200] {source.where}: {len(self.unused_tensors)} tensors the model does not use: "
                  + ", ".join(self.unused_tensors), file=sys.stderr, flush=True)
        self.model.bind(tensors)
        del tensors
        torch.cuda.synchronize(self.device)
        t1 = time.perf_counter()
        kernel_lib.preload(self.model.kernel_libraries())
        t2 = time.perf_counter()
        self._make_caches()
        torch.cuda.synchronize(self.device)
        self.startup_seconds = {"weights": t1 - t0, "kernels": t2 - t1, "caches": time.perf_counter() - t2}
        self.plan = PlanBuilder(self.manager, self.device,
                                max_tokens=engine.max_num_batched_tokens + engine.max_num_seqs,
                                max_reqs=engine.max_num_seqs + self.PROMPT_PLACES[-1],
                                max_blocks=self.max_blocks_per_seq, max_positions=self.spec.max_positions,
                                spare_state_slot=engine.max_num_seqs)
        # the tokens the last step sampled stay here (a fixed address, so that captured graphs can read it):
        # a step launched before the host has read them names them by row (see StepEntry.tokens)
        self.sampled = torch.zeros(max(1, engine.max_num_seqs), dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self._init_graphs()
        if self._graph_ok and engine.capture_graphs_at_start:
            for bucket in self._buckets:
                self._capture(bucket)

    @classmethod
    def from_dir(cls, model_dir: str, engine: EngineConfig) -> "ModelRunner":
        src = SafetensorsSource(model_dir)
        try:
            return cls(read_config_json(model_dir), src, engine)
        finally:
            src.close()

    # ---- caches
    def _make_caches(self) -> None:
        e = self.engine
        bs = e.block_size
        needs = self.model.cache_needs()
        group_keys: List[Any] = []
        entry_group: List[int] = []
        for n in needs:
            if isinstance(n, KvCacheNeed):
                key = n.group_key()
                if key not in group_keys:
                    group_keys.append(key)
                entry_group.append(group_keys.index(key))
            else:
                entry_group.append(-1)
        groups = [GroupSpec(window=k[1], block_size=k[2]) for k in group_keys]
        sizes = [k[2] or bs for k in group_keys]             # tokens a page of each group holds
        if any(b <= 0 for b in sizes):
            raise ValueError("a cache group's block_size must be positive")
        # one table width for all groups: what the group with the smallest pages needs
        self.max_blocks_per_seq = max([(e.max_model_len + b - 1) // b for b in sizes] or [(e.max_model_len + bs - 1) // bs])
        elt = 4 if self.act_dtype == torch.float32 else 2
        bytes_per_token = sum(2 * n.num_kv_heads * n.head_dim * elt for n in needs if isinstance(n, KvCacheNeed))
        # every group gets pages for the same number of tokens: ``num_blocks`` pages of the engine's page size
        longest = (e.max_model_len + bs - 1) // bs
        if e.num_blocks is not None:
            num_blocks = e.num_blocks
        else:
            free, total = torch.cuda.mem_get_info(self.device)
            used = total - free
            budget = min(free, int(total * e.gpu_memory_utilization) - used) - (2 << 30)
            num_blocks = max(0, budget // max(1, bytes_per_token * bs)) if bytes_per_token else 1
            if num_blocks < longest:
                raise RuntimeError(f"not enough device memory for the cache: room for {num_blocks} pages, "
                                   f"one request of max_model_len needs {longest}")
            # never more than every sequence at full length could use
            num_blocks = min(num_blocks, longest * e.max_num_seqs)
        self.num_blocks = int(num_blocks)
        group_blocks = [max(1, self.num_blocks * bs // b) for b in sizes]
        prefix = bool(e.enable_prefix_caching)
        if prefix and (any(g.window is not None for g in groups) or any(isinstance(n, StateNeed) for n in needs)):
            raise ValueError("enable_prefix_caching: this model has windowed layers or per-request state, "
                             "whose cache cannot be shared between requests")
        if e.native_host:
            from ..cache.native import NativeCacheManager as Manager
        else:
            Manager = CacheManager
        self.manager = Manager(groups, bs, group_blocks, e.max_num_seqs, enable_prefix_caching=prefix)
        self.bindings: List[CacheBinding] = []
        for i, (entry, n) in enumerate(zip(self.spec.schedule, needs)):
            if entry.cache_from is not None:
                src = self.bindings[entry.cache_from]
                self.bindings.append(CacheBinding(kv=src.kv, group=src.group, write=False, state=src.state))
            elif isinstance(n, KvCacheNeed):
                g = entry_group[i]
                kv = torch.zeros((group_blocks[g], 2, n.num_kv_heads, sizes[g], n.head_dim),
                                 dtype=self.act_dtype, device=self.device)
                self.bindings.append(CacheBinding(kv=kv, group=entry_group[i], write=True))
            elif isinstance(n, StateNeed):
                # one slot more than requests: the rows that pad a captured batch point at it
                st = torch.zeros((e.max_num_seqs + 1,) + tuple(n.shape), dtype=n.dtype, device=self.device)
                self.bindings.append(CacheBinding(state=st, group=-1, write=True))
            else:
                self.bindings.append(CacheBinding())

    # ---- one step
    def step(self, entries: Sequence[StepEntry], placeholders: bool = False) -> torch.Tensor:
        """``placeholders``: a token id -(r + 1) is allowed and stands for ``self.sampled[r]``, the token that
        row r of the previous step's sampling produced (still on the device)."""
        if not entries:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        m = self.manager
        seen = set()
        starts = []
        for e in entries:
            if e.req_id in seen:
                raise ValueError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.req_id!r} brings no token")
            if min(e.tokens) < (-self.sampled.numel() if placeholders else 0) or max(e.tokens) >= self.spec.vocab_size:
                raise ValueError(f"request {e.req_id!r}: a token id is outside the vocabulary "
                                 f"[0, {self.spec.vocab_size})")
            start = m.num_computed(e.req_id) if e.req_id in m else 0
            total = start + len(e.tokens)
            if total > self.engine.max_model_len:
                raise ValueError(f"request {e.req_id!r} would reach {total} tokens, max_model_len is "
                                 f"{self.engine.max_model_len}")
            starts.append(start)
        # all or nothing: a step that does not fit leaves every table and state slot as it was
        totals = [(e.req_id, s + len(e.tokens)) for e, s in zip(entries, starts)]
        if not m.can_allocate_all(totals):
            raise OutOfPages(f"no pages for this step of {len(entries)} requests growing to "
                             f"{[t for _, t in totals]} tokens ({[p.num_free for p in m.pools]} pages free, "
                             f"{m.state_slots.num_free} state slots free)")
        for rid, total in totals:
            if not m.allocate(rid, total):
                raise RuntimeError(f"request {rid!r}: the cache manager refused pages it had promised")
        mixed = None
        if self._graph_ok and len(entries) <= self._buckets[-1] and all(len(e.tokens) == 1 for e in entries):
            logits = self._graph_step(entries, starts)
        elif self._graph_ok and (mixed := self._mixed_layout(entries, starts)) is not None:
            logits = self._mixed_graph_step(entries, starts, *mixed)
        else:
            ids, rows, ctx = self.plan.build(entries, starts)
            ctx.split_norms = self.engine.split_norms is True
            ctx.prev_tokens = self.sampled
            logits = self.model.forward(ids, ctx, self.bindings, rows)
        for e, s in zip(entries, starts):
            m.advance(e.req_id, s + len(e.tokens), e.tokens if m.prefix_caching else None)
        self.steps_run += 1
        return logits

    # ---- decode-only steps replay a captured graph
    def _init_graphs(self) -> None:
        """Decode-only steps (every request brings one token) run as a CUDA graph per batch-size
        bucket, the batch padded with dummy rows up to the bucket (models/qwen3/src/executor.rs:993-1023,
        crates/layers/src/exec.rs:83-87).  A model with per-request state replays graphs too if every mixer with
        state says its forward can be captured (``Mixer.graph_capturable``); the dummy rows share a spare state slot."""
        e = self.engine
        self._graph_ok = bool(e.enable_cuda_graph) and self.model.graph_capturable()
        b, buckets = 1, []
        while b < e.max_num_seqs:
            buckets.append(b)
            b *= 2
        buckets.append(e.max_num_seqs)
        self._buckets = buckets
        self._graphs: Dict[Any, Any] = {}
        self._graph_pool = None
        self._mixed_seen: Dict[Any, int] = {}
        self._padded_tokens = self._padded_limit()

    def _capture(self, bucket: int):
        from ..kernels import attention_ops
        width = self.max_blocks_per_seq
        dev = torch.empty(self.plan.words(bucket, bucket, bucket, width), dtype=torch.int32, device=self.device)
        ids, rows, ctx = self.plan.build([], [], pad_reqs=bucket, table_width=width, dev=dev)
        # the split count is part of the captured launch: fixed per bucket, for the longest context
        hkv = max([n.num_kv_heads for n in self.model.cache_needs() if isinstance(n, KvCacheNeed)] or [1])
        ctx.decode_splits = attention_ops.decode_splits(bucket, hkv, self.engine.max_model_len)
        ctx.split_norms = self.engine.split_norms is True
        ctx.prev_tokens = self.sampled
        rec = self._capture_one(ids, rows, ctx)
        rec["split_norms"] = ctx.split_norms
        if self.engine.split_norms == "auto" and self.model.can_split_norms(bucket):
            # both forms of the step, measured on this device: the one with the norms taken apart where it is faster
            apart = self._capture_one(ids, rows, dataclasses.replace(ctx, split_norms=True, derived={}))
            t_whole, t_apart = self._graph_time(rec["graph"]), self._graph_time(apart["graph"])
            if t_apart <= 0.98 * t_whole:
                rec = apart
                rec["split_norms"] = True
            rec["times_ms"] = (t_whole, t_apart)
        rec.update(dev=dev, splits=ctx.decode_splits, width=width, plan=DecodePlan(self.plan, bucket, width, dev))
        self._graphs[bucket] = rec
        return rec

    @staticmethod
    def _graph_time(graph, replays: int = 8, rounds: int = 3) -> float:
        """Milliseconds per replay: the best of a few rounds of back-to-back replays between CUDA events."""
        graph.replay()
        best = None
        for _ in range(rounds):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(replays):
                graph.replay()
            e1.record()
            e1.synchronize()
            ms = e0.elapsed_time(e1) / replays
            best = ms if best is None else min(best, ms)
        return best

    def split_norms_buckets(self) -> List[int]:
        """The decode buckets captured so far whose graph runs with the norms taken apart."""
        return sorted(k for k, r in self._graphs.items() if isinstance(k, int) and r.get("split_norms"))

    def _capture_one(self, ids, rows, ctx):
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(2):                               # warm-up outside the capture
                self.model.forward(ids, ctx, self.bindings, rows)
        cur.wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = kernel_lib.launch_count()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self.model.forward(ids, ctx, self.bindings, rows)
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        return dict(graph=graph, logits=logits, launches=kernel_lib.launch_count() - n0)

    def _graph_step(self, entries: Sequence[StepEntry], starts: Sequence[int]) -> torch.Tensor:
        B = len(entries)
        bucket = next(b for b in self._buckets if b >= B)
        rec = self._graphs.get(bucket) or self._capture(bucket)
        rec["plan"].fill(entries, starts)
        rec["graph"].replay()
        self._last_graph = rec
        kernel_lib.add_launches(rec["launches"])
        wanted = [i for i, e in enumerate(entries) if len(e.want)]
        if len(wanted) == B:
            return rec["logits"][:B]         # valid until the next step of this bucket
        if not wanted:
            return rec["logits"][:0]
        return rec["logits"][torch.tensor(wanted, device=self.device)]

    # ---- steps with prompt portions replay a captured graph too where their shape comes again
    def _padded_limit(self) -> int:
        """The most prompt tokens of a step that is padded (up to a multiple of 128) to replay a graph: as long as
        launching the step kernel by kernel would keep the host busy for longer than the device needs for the
        padded step.  Both sides are estimates from the model's sizes, so the answer is the same in every run:
        ``EngineConfig.graph_host_us_per_layer`` for the host, two flops per weight and token at
        ``EngineConfig.graph_device_flops`` for the device."""
        table = (self.spec.vocab_size, self.spec.hidden_size)       # the table and the head do not see every row
        weights = sum(math.prod(d.shape) for d in self.model.declarations()
                      if len(d.shape) == 2 and tuple(d.shape) != table)
        host_s = len(self.spec.schedule) * self.engine.graph_host_us_per_layer * 1e-6
        tokens = int(host_s * self.engine.graph_device_flops / (2.0 * max(1, weights)))
        return max(self.PADDED_PROMPT_TOKENS, tokens // 128 * 128)

    def _mixed_layout(self, entries: Sequence[StepEntry], starts: Sequence[int]):
        """Steps with prompt portions whose shape comes again replay a graph per (prompt tokens, decode bucket), laid
        out as ``PROMPT_PLACES`` prompt places (a dummy portion that pads the prompt tokens in one of them, the
        unused ones without tokens) followed by the bucket's one-token places (the unused ones dummy rows):
          * portions that add up to exactly the token budget (the steady state while prompts are taken in);
          * at most ``PADDED_PROMPT_TOKENS`` prompt tokens, padded up to a power of two (so few rows cost a product
            nothing: it is bound by reading its weights);
          * more than that, padded up to a multiple of 128 (256 beyond 1024 tokens), for models small enough that
            the host would be the slower side of such a step (``_padded_limit``).
        Returns (key, places), or None for a step that runs kernel by kernel.  A shape is captured when it comes
        up the second time."""
        if not self.engine.mixed_cuda_graph:
            return None
        prompts = [i for i, e in enumerate(entries) if len(e.tokens) > 1]
        decodes = [i for i, e in enumerate(entries) if len(e.tokens) == 1]
        if any(tuple(e.want) not in ((), (len(e.tokens) - 1,)) for e in entries):
            return None                                      # only the last token's logits come out of a place
        shape = graph_shape([len(entries[i].tokens) for i in prompts], len(decodes),
                            self.engine.max_num_batched_tokens, self._buckets, self.PROMPT_PLACES,
                            self.PADDED_PROMPT_TOKENS, self._padded_tokens, longest=self.engine.max_model_len)
        if shape is None:
            return None
        total, n_places, bucket = shape
        have = sum(len(entries[i].tokens) for i in prompts)
        short = all(starts[i] + len(entries[i].tokens) <= self.SHORT_CONTEXT for i in prompts)
        key = ("mixed", total, n_places, bucket, short)
        if key not in self._graphs:
            self._mixed_seen[key] = self._mixed_seen.get(key, 0) + 1
            if self._mixed_seen[key] < 2:
                return None
        places = [(i, len(entries[i].tokens)) for i in prompts]
        if total > have:
            places.append((-1, total - have))
        places += [(-1, 0)] * (n_places - len(places))
        places += [(i, 1) for i in decodes] + [(-1, 1)] * (bucket - len(decodes))
        return key, places

    def _capture_mixed(self, key):
        from ..kernels import attention_ops
        _, total, n_places, bucket, short = key
        width = self.max_blocks_per_seq
        B = n_places + bucket
        dev = torch.empty(self.plan.words(total + bucket, B, B, width), dtype=torch.int32, device=self.device)
        # captured on a dummy batch of the same shape (no pages, no slots): the prompt tokens in as few places as
        # hold them without passing the longest request the tables and the position table are made for
        places = capture_places(total, n_places, bucket, self.engine.max_model_len)
        ids, rows, ctx = self.plan.build([], [], table_width=width, dev=dev, slots=places)
        hkv = max([n.num_kv_heads for n in self.model.cache_needs() if isinstance(n, KvCacheNeed)] or [1])
        ctx.decode_splits = attention_ops.decode_splits(max(1, bucket), hkv, self.engine.max_model_len)
        ctx.max_seq_len = self.engine.max_model_len
        ctx.max_prefill_seq_len = min(self.SHORT_CONTEXT, self.engine.max_model_len) if short else self.engine.max_model_len
        ctx.split_norms = False
        ctx.prev_tokens = self.sampled
        rec = self._capture_one(ids, rows, ctx)
        rec.update(dev=dev, width=width)
        self._graphs[key] = rec
        return rec

    def _mixed_graph_step(self, entries: Sequence[StepEntry], starts: Sequence[int], key, places) -> torch.Tensor:
        rec = self._graphs.get(key) or self._capture_mixed(key)
        self.plan.build(entries, starts, table_width=rec["width"], dev=rec["dev"], slots=places)
        rec["graph"].replay()
        kernel_lib.add_launches(rec["launches"])
        place_of = {i: j for j, (i, _) in enumerate(places) if i >= 0}
        wanted = [place_of[i] for i, e in enumerate(entries) if len(e.want)]
        if not wanted:
            return rec["logits"][:0]
        return rec["logits"][torch.tensor(wanted, device=self.device)]

    def replay_last_decode(self, times: int = 1, after=None) -> int:
        """Replay the decode graph of the last decode-only step ``times`` more times with the same
        batch (same tokens, positions and pages: the step's device work again, nothing advances).
        For measuring the device time of one decode step without the host between steps.  Returns the
        kernel launches replayed."""
        rec = getattr(self, "_last_graph", None)
        if rec is None:
            raise RuntimeError("no decode-only step has run through a CUDA graph yet")
        for _ in range(times):
            rec["graph"].replay()
            if after is not None:
                after(rec["logits"])                  # e.g. the sampling kernel, launched behind the graph
        kernel_lib.add_launches(rec["launches"] * times)
        return rec["launches"] * times

    def check_device_status(self) -> None:
        """Raise if a kernel recorded a fault in its status word (a bounded wait that ran out).
        Reading the word synchronizes with the device."""
        from ..kernels import gemm_ops
        gemm_ops.check_status(self.device)

    def reset_device_status(self) -> int:
        """Clear the status word after a reported fault; returns the code it held."""
        from ..kernels import gemm_ops
        return gemm_ops.reset_status(self.device)

    def finish(self, req_id: Hashable) -> None:
        """The request is over: its pages and state slot go back to the pools."""
        if req_id in self.manager:
            self.manager.free(req_id)
