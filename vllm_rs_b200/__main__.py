"""Command line of the package.

    python -m vllm_rs_b200 generate --model DIR --prompt-ids 1,2,3 [--prompt-ids ...] [--max-new-tokens N]
                                    [--dtype bfloat16|float32|float16] [--temperature T --top-k K --top-p P --seed S]
    python -m vllm_rs_b200 trace    --model DIR --dtype ... --out DIR --max-tokens N      (bin/trace_run)
    python -m vllm_rs_b200 models                                                       (registered architectures)

`generate` loads a model folder (config.json + *.safetensors) through the model registry and runs the prompts, given
as token ids (there is no tokenizer on this path), through LLMEngine: scheduler, block manager, state slots, the
runner's step function and the device sampler.  It prints one JSON line per request."""
from __future__ import annotations

import argparse
import json
import sys


def _generate(a) -> int:
    import torch

    from . import _lib, build, engine, models, ops
    from .weights import read_model_dir
    cfg, tensors = read_model_dir(a.model)
    arch = models.architecture_of(cfg)
    if not _lib.LIB_PATH.exists() and not _lib.HYBRID_LIB_PATH.exists():
        build.build(verbose=False, target="hybrid" if arch in models.HYBRID_ARCHITECTURES else "full")
    prompts = [[int(x) for x in p.split(",") if x.strip()] for p in a.prompt_ids]
    longest = max(len(p) for p in prompts) + a.max_new_tokens
    per_seq = (longest + 63) // 64 + 2
    n = max(len(prompts), 1)
    num_blocks = per_seq * n + 2          # the block manager keeps a spare block per appending sequence
    dtype = getattr(torch, a.dtype) if a.dtype else None
    runner = models.build_runner(cfg, tensors, dtype=dtype, device="cuda", num_blocks=num_blocks,
                                 max_blocks_per_seq=per_seq, max_seqs=max(n, 5), max_tokens=a.chunk,
                                 num_state_slots=max(n, 5))
    strat, k, p, t = ops.sampling_strategy(a.temperature, a.top_k, a.top_p)
    if hasattr(runner, "step"):
        runner.set_sampling(strat, k, p, t)
    elif strat:
        runner._l.b200_runner_set_sampling_strategy(runner._h, strat, k, p, t)
    eng = engine.LLMEngine(runner, num_blocks, max(n, 1), eos_token_ids=a.eos, chunk_size=a.chunk,
                           seed=a.seed if strat else None, native_step=False)
    sids = [eng.add_request(p, a.max_new_tokens) for p in prompts]
    out = eng.run_to_completion()
    for sid, p in zip(sids, prompts):
        print(json.dumps({"prompt_ids": p, "output_ids": out[sid]}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m vllm_rs_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate")
    g.add_argument("--model", required=True)
    g.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeatable")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--dtype", default=None, choices=["bfloat16", "float32", "float16"])
    g.add_argument("--chunk", type=int, default=2048, help="prompt tokens per prefill step")
    g.add_argument("--temperature", type=float, default=None)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--top-p", type=float, default=None)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--eos", type=int, action="append", default=[])
    t = sub.add_parser("trace")
    t.add_argument("rest", nargs=argparse.REMAINDER)
    sub.add_parser("models")
    a = ap.parse_args(argv)
    if a.cmd == "trace":
        from . import trace_run
        return trace_run.main(a.rest)
    if a.cmd == "models":
        from . import models
        print("\n".join(models.registered()))
        return 0
    return _generate(a)


if __name__ == "__main__":
    sys.exit(main())
