"""Trace runner: replays given token ids through a model step by step and writes logits; it samples nothing.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps arrive on standard input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
All entries of a step run as ONE ragged batch through the engine's own pieces: the scheduler's block manager and
state slots (streamed sequences: open / feed / close), b200_prepare_ragged, and the runner's step function.  A request
is admitted at its first entry; `want` lists the places among the step's tokens whose logits are written, in order,
to DIR/<step>.f32 (little-endian fp32 [wanted, vocab]); `end` closes requests after the step, which returns their
pages and slot.  After every step the line "done <step>" is printed.  The cache pool holds --max-tokens tokens
(whole 64-token pages), and there are state slots for four live requests.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

MAX_LIVE = 4


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run")
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    a = ap.parse_args(argv)

    from . import _lib, build
    if not _lib.LIB_PATH.exists() and not _lib.HYBRID_LIB_PATH.exists():
        build.build(verbose=False, target="hybrid")      # a fresh checkout compiles what this family needs
    import numpy as np
    import torch

    from . import engine, models
    from .weights import read_model_dir

    cfg, tensors = read_model_dir(a.model)
    page = 64
    num_blocks = (a.max_tokens + page - 1) // page
    runner = models.build_runner(cfg, tensors, dtype=getattr(torch, a.dtype), device="cuda", num_blocks=num_blocks,
                                 max_blocks_per_seq=num_blocks, max_seqs=MAX_LIVE, max_tokens=num_blocks * page,
                                 num_state_slots=MAX_LIVE)
    if not hasattr(runner, "step"):
        print("this model family has no ragged-step runner", file=sys.stderr)
        return 3
    del tensors
    sched = engine.Scheduler(num_blocks, page, MAX_LIVE, 0, num_blocks * page)
    sched.enable_state_slots(MAX_LIVE)
    os.makedirs(a.out, exist_ok=True)
    live: dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        ids, rows, base = [], [], 0
        for e in step["entries"]:
            if e["id"] not in live:
                sid = sched.open()
                if sid < 0:
                    raise RuntimeError("no free state slot for a new request")
                live[e["id"]] = sid
            rc = sched.feed(live[e["id"]], e["tokens"])
            if rc != 0:
                raise RuntimeError("the cache pool has no page left for this step" if rc == -1 else "bad entry")
            ids.append(sched.running_index(live[e["id"]]))
            rows += [base + int(w) for w in e.get("want", [])]
            base += len(e["tokens"])
        if ids:
            meta = sched.prepare_ragged(ids, None, 2, runner.cfg.max_tokens, num_blocks, pinned=runner.pinned)
            logits, _ = runner.step(meta, rows, want_logits=True, want_ids=False)
            if rows:
                tmp = os.path.join(a.out, f".{step['step']}.part")
                np.ascontiguousarray(logits, dtype="<f4").tofile(tmp)
                os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        for rid in step.get("end", []):
            if rid in live:
                sched.close(live.pop(rid))
        print(f"done {step['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
