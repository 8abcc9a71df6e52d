"""Command line, in the manner of the reference's ``dinfer`` binary (bins/dinfer/src/main.rs:28-151):
sub-commands, and for the engine options the reference's own flag names and defaults
(``--model --max-model-len --max-num-seqs --max-num-batched-tokens --num-blocks --block-size
--gpu-memory-utilization --no-cuda-graph --no-mixed-cuda-graph --enable-prefix-caching --split-norms
--no-async-scheduling --no-decode-exempt --long-prefill-token-threshold --device``).  The reference serves HTTP; this engine starts at token ids, so ``generate`` takes the
place of ``serve``:

    dinfer generate --model DIR --prompt-ids 1,2,3 --prompt-ids 4,5 --max-tokens 16 --temperature 0
    dinfer generate --random-weights config.json --weights-seed 0 --prompt-ids 1,2,3     (no files: weights made on the device)
    dinfer random-model --config config.json --out DIR --seed 0
    dinfer device-info
    dinfer replay --model DIR --dtype bfloat16 --out DIR --max-tokens N < steps.jsonl     (= bin/trace_run)
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List


def _engine_flags(p: argparse.ArgumentParser) -> None:
    src = p.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="model folder (config.json + safetensors)")
    src.add_argument("--random-weights", metavar="CONFIG_JSON",
                     help="no model folder: the architecture and every size from this config.json, the weights drawn "
                          "on the device (see --weights-seed, --weights-std, --weights-norm-jitter)")
    p.add_argument("--weights-seed", type=int, default=0, help="with --random-weights: the seed of the weights")
    p.add_argument("--weights-std", type=float, default=0.02, help="with --random-weights: matrices are N(0, std)")
    p.add_argument("--weights-norm-jitter", type=float, default=0.0,
                   help="with --random-weights: norm weights are 1 + U(-jitter, jitter)")
    p.add_argument("--allow-unused-tensors", action="store_true",
                   help="tensors in the model's files that the model does not use are reported, not refused")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--max-model-len", type=int, default=4096)
    p.add_argument("--max-num-seqs", type=int, default=16)
    p.add_argument("--max-num-batched-tokens", type=int, default=2048)
    p.add_argument("--num-blocks", type=int, default=None, help="cache pages; default: from free device memory")
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    p.add_argument("--no-decode-exempt", action="store_true",
                   help="decoded tokens count against the token budget")
    p.add_argument("--long-prefill-token-threshold", type=int, default=0)
    p.add_argument("--no-cuda-graph", action="store_true")
    p.add_argument("--enable-prefix-caching", action="store_true",
                   help="share the cached pages of equal prompt beginnings between requests")
    p.add_argument("--split-norms", nargs="?", const="on", default="off", choices=["on", "off", "auto"],
                   help="decode steps: take the RMSNorms between two products apart into the products' epilogues; "
                        "auto = measured per batch-size bucket when its graph is captured (see EngineConfig.split_norms)")
    p.add_argument("--no-mixed-cuda-graph", action="store_true",
                   help="steps with prompt portions always launch their kernels one by one")
    p.add_argument("--no-async-scheduling", action="store_true",
                   help="read every step's tokens before the next step is scheduled (default: one step in flight)")
    p.add_argument("--device", type=int, default=0)


def _ids(text: str) -> List[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def cmd_generate(a) -> int:
    from .. import LLM, SamplingParams
    prompts = [_ids(t) for t in (a.prompt_ids or [])]
    if a.prompt_file:
        with open(a.prompt_file) as f:
            for line in f:
                line = line.strip()
                if line:
                    prompts.append(json.loads(line) if line.startswith("[") else _ids(line))
    if not prompts:
        print("no prompt given (--prompt-ids or --prompt-file)", file=sys.stderr)
        return 2
    source = {}
    if a.random_weights:
        import torch
        from ..weights.random_init import RandomSource
        with open(a.random_weights) as f:
            cfg = json.load(f)
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[a.dtype]
        source = dict(config=cfg, weights=RandomSource(cfg, a.weights_seed, a.weights_std, a.weights_norm_jitter, dt,
                                                       device=f"cuda:{a.device}"))
    llm = LLM(a.model, **source, allow_unused_tensors=a.allow_unused_tensors, dtype=a.dtype, max_model_len=a.max_model_len, max_num_seqs=a.max_num_seqs,
              max_num_batched_tokens=a.max_num_batched_tokens, num_blocks=a.num_blocks,
              block_size=a.block_size, gpu_memory_utilization=a.gpu_memory_utilization,
              decode_exempt_from_budget=not a.no_decode_exempt,
              long_prefill_token_threshold=a.long_prefill_token_threshold,
              enable_cuda_graph=not a.no_cuda_graph, enable_prefix_caching=a.enable_prefix_caching, split_norms={"on": True, "off": False, "auto": "auto"}[a.split_norms],
              async_scheduling=not a.no_async_scheduling, mixed_cuda_graph=not a.no_mixed_cuda_graph,
              device=a.device)
    su = llm.runner.startup_seconds
    print(f"start-up: weights {su['weights']:.2f} s  kernels {su['kernels']:.2f} s  caches {su['caches']:.2f} s  "
          f"({llm.runner.num_blocks} pages of {llm.engine_config.block_size} tokens)", file=sys.stderr)
    d = llm.default_sampling_params
    sp = SamplingParams(max_tokens=a.max_tokens, min_tokens=a.min_tokens,
                        temperature=d.temperature if a.temperature is None else a.temperature,
                        top_p=d.top_p if a.top_p is None else a.top_p,
                        top_k=d.top_k if a.top_k is None else a.top_k, min_p=a.min_p,
                        repetition_penalty=a.repetition_penalty, frequency_penalty=a.frequency_penalty,
                        presence_penalty=a.presence_penalty, seed=a.seed,
                        stop_token_ids=_ids(a.stop_token_ids) if a.stop_token_ids else [],
                        ignore_eos=a.ignore_eos, logprobs=a.logprobs, prompt_logprobs=a.prompt_logprobs,
                        logit_bias={int(t): float(b) for t, b in
                                    (x.split(":") for x in a.logit_bias.replace(",", " ").split())})
    for o in llm.generate(prompts, sp):
        rec = {"id": o.req_id, "output_ids": o.output_ids, "finish_reason": o.finish_reason,
               "ttft_ms": round(o.ttft_s * 1e3, 3), "tpot_ms": round(o.tpot_s * 1e3, 3), "e2e_ms": round(o.e2e_s * 1e3, 3)}
        if o.prompt_logprobs is not None:
            rec["prompt_logprobs"] = [None if t is None else {"token_id": t.token_id, "logprob": t.logprob, "rank": t.rank,
                                                             "top": list(zip(t.top_ids, t.top_logprobs))}
                                      for t in o.prompt_logprobs]
        if o.logprobs is not None:
            rec["logprobs"] = [{"token_id": t.token_id, "logprob": t.logprob, "rank": t.rank,
                                "top": list(zip(t.top_ids, t.top_logprobs))} for t in o.logprobs]
        print(json.dumps(rec))
    s = llm.stats
    print(f"steps {s.steps}  prompt tokens {s.prompt_tokens}  generated {s.generated_tokens}  "
          f"preemptions {s.preemptions}  prefix hits {s.prefix_hit_tokens}", file=sys.stderr)
    if s.steps:
        print(f"host time per step: schedule {s.host_schedule_s / s.steps * 1e6:.0f} us  plan and launch "
              f"{s.host_launch_s / s.steps * 1e6:.0f} us  wait for and apply tokens {s.host_collect_s / s.steps * 1e6:.0f} us",
              file=sys.stderr)
    return 0


def cmd_random_model(a) -> int:
    import torch
    from ..weights.random_init import write_random_model
    with open(a.config) as f:
        cfg = json.load(f)
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[a.dtype]
    write_random_model(a.out, cfg, a.seed, a.std, a.norm_jitter, dt)
    print(a.out)
    return 0


def cmd_device_info(a) -> int:
    import torch
    if not torch.cuda.is_available():
        print("no CUDA device")
        return 1
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        free, total = torch.cuda.mem_get_info(i)
        print(json.dumps({"index": i, "name": p.name, "compute_capability": f"{p.major}.{p.minor}",
                          "multiprocessors": p.multi_processor_count, "memory_total": total,
                          "memory_free": free}))
    return 0


def cmd_replay(rest) -> int:
    import os
    import runpy
    script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "bin", "trace_run")
    sys.argv = [script] + list(rest)
    try:
        runpy.run_path(script, run_name="__main__")
    except SystemExit as e:
        return int(e.code or 0)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":                     # everything behind it belongs to trace_run
        return cmd_replay(argv[1:])
    ap = argparse.ArgumentParser(prog="dinfer", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    _engine_flags(g)
    g.add_argument("--prompt-ids", action="append", help="comma separated token ids; may repeat")
    g.add_argument("--prompt-file", help="one prompt a line: JSON list or separated ids")
    g.add_argument("--max-tokens", type=int, default=256)
    g.add_argument("--min-tokens", type=int, default=0)
    g.add_argument("--temperature", type=float, default=None,
                   help="default: the model folder's generation_config.json, else 1.0 (the same for --top-p, 1.0, "
                        "and --top-k, -1 = off)")
    g.add_argument("--top-p", type=float, default=None)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--stop-token-ids", default="")
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--logprobs", type=int, default=None,
                   help="with every generated token: its log-probability, its rank and this many most likely tokens")
    g.add_argument("--prompt-logprobs", type=int, default=None,
                   help="with every prompt token but the first: its log-probability given the tokens before it, its "
                        "rank and this many most likely tokens")
    g.add_argument("--logit-bias", default="", help="TOKEN:BIAS pairs, comma separated, added to the logits")
    g.set_defaults(fn=cmd_generate)
    r = sub.add_parser("random-model", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="a config.json")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--norm-jitter", type=float, default=0.0)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.set_defaults(fn=cmd_random_model)
    d = sub.add_parser("device-info", help="list the CUDA devices")
    d.set_defaults(fn=cmd_device_info)
    sub.add_parser("replay", help="trace replay: the arguments and the standard input of bin/trace_run",
                   add_help=False)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
