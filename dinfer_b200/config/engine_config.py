"""Engine options, with the names and meanings of the reference's ``ServeOptions``
(models/qwen3/src/service.rs:43-140) and of its ``dinfer serve`` flags
(bins/dinfer/src/main.rs:30-131) where it has them."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional


@dataclass
class EngineConfig:
    # longest sequence (prompt + generated) a request may reach
    max_model_len: int = 4096
    # most requests running at the same time
    max_num_seqs: int = 16
    # token budget of one step; a longer prompt is cut into portions of at most this many
    max_num_batched_tokens: int = 2048
    # pages of the cache pool; None = from the free device memory
    num_blocks: Optional[int] = None
    # tokens per page
    block_size: int = 16
    # share of the device memory that weights, scratch and cache may take together
    gpu_memory_utilization: float = 0.9
    # decoded tokens do not count against the token budget (so every running request decodes
    # in every step and prompts fill what is left)
    decode_exempt_from_budget: bool = True
    # one prompt gets at most this many tokens a step (0 = no limit)
    long_prefill_token_threshold: int = 0
    # decode-only steps replay a captured CUDA graph
    enable_cuda_graph: bool = True
    # the decode graphs of every batch-size bucket are captured when the engine starts, so that no request meets a
    # capture (some tens of milliseconds, now and then hundreds) in the middle of its decoding; off: each bucket's
    # graph is captured when a step first needs it
    capture_graphs_at_start: bool = True
    # steps whose prompt portions fill the token budget exactly (the steady state while prompts are taken in) and
    # steps with at most 128 prompt tokens (padded up to a power of two) replay a captured graph as well, one per
    # shape and bucket of decoded tokens beside them; pays where launching a step's kernels one by one takes the
    # host longer than the device needs to run them (small models, short prompts)
    mixed_cuda_graph: bool = True
    # the two estimates that decide up to how many prompt tokens a step is padded to replay a graph: what launching
    # one layer's kernels one by one costs the host (microseconds; measured through the Python wrappers) and what a
    # prompt-sized step reaches on the device (flops a second).  Fixed numbers, not measurements at start-up, so
    # that every run of a workload decides the same way
    graph_host_us_per_layer: float = 120.0
    graph_device_flops: float = 1.2e15
    # full pages of computed tokens stay findable by the hash of their tokens and are shared by later
    # requests with the same beginning (off by default: with it on, freed pages are not the next ones used)
    enable_prefix_caching: bool = False
    # RMSNorms between two decode products (steps of at most 32 rows, bfloat16): True = taken apart into the
    # products' epilogues wherever the parts can (two launches per layer less), False = kernels of their own.
    # Off by default: it pays here and costs there with no rule to it (closed loops of 128 + 128 tokens: +8 % at
    # the 0.6B shape with one client, -8 % with 32; -8 % at the 8B shape with one client, +3 % with 8).
    # "auto" = measured: every decode graph is captured in both forms when it is made, each is replayed a few
    # times between CUDA events, and the form taken apart is kept where it is faster by 2 % or more.  Steps that
    # run kernel by kernel keep the norms whole.  The two forms differ by roundings, so with "auto" the same seed
    # may give another text after a restart should a measurement fall the other way; hence not the default.
    split_norms: Any = False
    # the next step is scheduled and launched while the last one still runs; the host reads a step's tokens one
    # step late (the reference's ASYNC_SCHED, on by default there too: crates/core/src/engine.rs:153,822).
    # Steps with penalties or log-probabilities (which need the last tokens on the host) run one at a time
    # whatever this says.
    async_scheduling: bool = True
    # the cache manager's bookkeeping and the packed plan of decode steps in C++ (csrc/host_core.cpp) instead of
    # Python: the same decisions, fewer microseconds a step at large batches
    native_host: bool = True
    # tensors in the model's files that the model does not use: False = an error that lists them (with everything
    # else that does not fit); True = reported on the standard error stream and left alone
    allow_unused_tensors: bool = False
    # "bfloat16" = what serving uses; "float32" = everything in true 32-bit
    dtype: str = "bfloat16"
    device: int = 0

    def check(self) -> None:
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        if self.block_size <= 0:
            raise ValueError(f"block_size must be positive, got {self.block_size}")
        if self.max_num_seqs <= 0:
            raise ValueError(f"max_num_seqs must be positive, got {self.max_num_seqs}")
        if self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_batched_tokens must be positive")
        if self.max_model_len <= 1:
            raise ValueError("max_model_len must be at least 2")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.graph_host_us_per_layer < 0 or self.graph_device_flops <= 0:
            raise ValueError("graph_host_us_per_layer must not be negative and graph_device_flops must be positive")
        if self.split_norms not in (False, True, "auto"):
            raise ValueError(f'split_norms must be False, True or "auto", got {self.split_norms!r}')
        if self.num_blocks is not None and self.num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
