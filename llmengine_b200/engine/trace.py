"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: every step is one
call of `Engine.step`, the step function that generation uses.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, `<out>/<step>.f32` receives the logits at the
wanted places, in the order of the entries and of `want`, as little-endian 32-bit floats
[wanted, vocab].  After every step the line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

import numpy as np


def main(argv: Optional[List[str]] = None) -> int:
    from ..config import EngineConfig

    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (the cache pool is made for this many)")
    ap.add_argument("--page-size", type=int, default=EngineConfig().page_size)
    ap.add_argument("--max-requests", type=int, default=8, help="requests that may be live at once")
    ap.add_argument("--kernels", choices=["fast", "plain"], default="fast")
    args = ap.parse_args(argv)

    from .engine import Engine, StepEntry, StepError

    os.makedirs(args.out, exist_ok=True)
    page = args.page_size
    pool = max(page, -(-args.max_tokens // page) * page)
    ec = EngineConfig(dtype=args.dtype, page_size=page, max_cached_tokens=pool, max_num_seqs=args.max_requests,
                      max_num_batched_tokens=pool, prefill_chunk=pool, use_cuda_graphs=False, kernels=args.kernels)
    engine = Engine(args.model, engine_config=ec)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        try:
            rec = json.loads(line)
            step = rec["step"]
            entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
            end = rec.get("end", [])
        except (json.JSONDecodeError, KeyError, TypeError) as e:
            print(f"trace_run: bad input line: {e}: {line[:200]}", file=sys.stderr)
            return 2
        try:
            logits = engine.step(entries, end)
        except StepError as e:
            print(f"trace_run: step {step} refused: {e}", file=sys.stderr)
            return 3
        if logits is not None and logits.shape[0] > 0:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            arr.tofile(os.path.join(args.out, f"{step}.f32"))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
