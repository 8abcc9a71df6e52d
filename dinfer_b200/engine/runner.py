"""The step function.

``ModelRunner.step(entries)`` takes a batch of (request, its next tokens, wanted places): portions of
prompts beside single decoded tokens, cut anywhere.  It allocates pages for the new tokens, runs
only those tokens as one batch against the cache that earlier steps left, and returns the f32 logits
at the wanted places ``[R, V]`` (device tensor, in the order of the entries and of their ``want``).
Generation (scheduler + sampling) and trace replay both drive this one function.

It stands where the reference has ``Runner::execute`` -> ``Qwen3Executor::forward_sample`` ->
``Qwen3Model::forward`` (crates/core/src/runner.rs:362-429, models/qwen3/src/executor.rs:977-1026,
models/qwen3/src/model.rs:684-832), with sampling kept out of it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
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
from .batch import OutOfPages, PlanBuilder, StepEntry

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class ModelRunner:
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
        self.act_dtype = _TORCH_DTYPE[engine.dtype]
        arch = resolve_architecture(config_dict)
        self.config = arch.parse_config(config_dict)
        self.spec = arch.build_spec(self.config)
        if engine.max_model_len > self.spec.max_positions:
            raise ValueError(f"max_model_len {engine.max_model_len} exceeds the model's "
                             f"max_position_embeddings {self.spec.max_positions}")
        env = BuildEnv(self.device, self.act_dtype, self.spec.hidden_size, self.spec.max_positions)
        self.model = DecoderModel(self.spec, env)
        tensors = load_tensors(source, self.model.declarations(), self.act_dtype, self.device)
        self.model.bind(tensors)
        del tensors
        kernel_lib.preload(self.model.kernel_libraries())
        self._make_caches()
        self.plan = PlanBuilder(self.manager, self.device,
                                max_tokens=engine.max_num_batched_tokens + engine.max_num_seqs,
                                max_reqs=engine.max_num_seqs,
                                max_blocks=self.max_blocks_per_seq)
        self.steps_run = 0

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
        groups = [GroupSpec(window=k[1]) for k in group_keys]
        self.max_blocks_per_seq = (e.max_model_len + bs - 1) // bs
        elt = 4 if self.act_dtype == torch.float32 else 2
        bytes_per_block = sum(2 * n.num_kv_heads * bs * n.head_dim * elt
                              for n in needs if isinstance(n, KvCacheNeed))
        if e.num_blocks is not None:
            num_blocks = e.num_blocks
        else:
            free, total = torch.cuda.mem_get_info(self.device)
            used = total - free
            budget = min(free, int(total * e.gpu_memory_utilization) - used) - (2 << 30)
            num_blocks = max(0, budget // max(1, bytes_per_block * 1)) if bytes_per_block else 1
            if num_blocks < self.max_blocks_per_seq:
                raise RuntimeError(f"not enough device memory for the cache: room for {num_blocks} pages, "
                                   f"one request of max_model_len needs {self.max_blocks_per_seq}")
            # never more than every sequence at full length could use
            num_blocks = min(num_blocks, self.max_blocks_per_seq * e.max_num_seqs)
        self.num_blocks = int(num_blocks)
        self.manager = CacheManager(groups, bs, [self.num_blocks] * len(groups), e.max_num_seqs)
        self.bindings: List[CacheBinding] = []
        for i, (entry, n) in enumerate(zip(self.spec.schedule, needs)):
            if entry.cache_from is not None:
                src = self.bindings[entry.cache_from]
                self.bindings.append(CacheBinding(kv=src.kv, group=src.group, write=False, state=src.state))
            elif isinstance(n, KvCacheNeed):
                kv = torch.zeros((self.num_blocks, 2, n.num_kv_heads, bs, n.head_dim),
                                 dtype=self.act_dtype, device=self.device)
                self.bindings.append(CacheBinding(kv=kv, group=entry_group[i], write=True))
            elif isinstance(n, StateNeed):
                st = torch.zeros((e.max_num_seqs,) + tuple(n.shape), dtype=n.dtype, device=self.device)
                self.bindings.append(CacheBinding(state=st, group=-1, write=True))
            else:
                self.bindings.append(CacheBinding())

    # ---- one step
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
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
            if min(e.tokens) < 0 or max(e.tokens) >= self.spec.vocab_size:
                raise ValueError(f"request {e.req_id!r}: a token id is outside the vocabulary "
                                 f"[0, {self.spec.vocab_size})")
            start = m.num_computed(e.req_id) if e.req_id in m else 0
            total = start + len(e.tokens)
            if total > self.engine.max_model_len:
                raise ValueError(f"request {e.req_id!r} would reach {total} tokens, max_model_len is "
                                 f"{self.engine.max_model_len}")
            if not m.allocate(e.req_id, total):
                raise OutOfPages(f"no pages for request {e.req_id!r} ({total} tokens; "
                                 f"{[p.num_free for p in m.pools]} pages free)")
            starts.append(start)
        ids, rows, ctx = self.plan.build(entries, starts)
        logits = self.model.forward(ids, ctx, self.bindings, rows)
        for e, s in zip(entries, starts):
            m.advance(e.req_id, s + len(e.tokens))
        self.steps_run += 1
        return logits

    def finish(self, req_id: Hashable) -> None:
        """The request is over: its pages and state slot go back to the pools."""
        if req_id in self.manager:
            self.manager.free(req_id)
