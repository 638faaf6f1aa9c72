"""Command line in the manner of the reference's `generate`
(examples/generate.cpp:57-65: `generate <model.gguf> [prompt] [max_tokens]`, prompt "Hello",
max_tokens 64, greedy, progress on stderr, result on stdout, `[Generated N tokens total]`).

    python -m llmengine_b200.generate <model_dir> [prompt] [max_tokens] [options]
    python -m llmengine_b200.generate --random-config config.json --seed 7 [prompt] [max_tokens] [options]

This engine works on token ids (it has no tokenizer), so `prompt` is a list of ids separated by
commas or spaces, default "1".  Several prompts may be given separated by ';', or one a line in
a file (`--prompt-ids-file`).  The sampling options carry the names of the reference's
SamplingConfig fields.  With `--random-config` the model is a config.json alone: its weights are
drawn from `--seed` (the folder that `python -m llmengine_b200.make_random_model` would write,
made in a temporary place).  `--print-logits N` also prints, for each prompt, the N largest
logits at its last prompt token (token:value pairs), which the reference's Sampler::get_top_tokens
gives (src/runtime/sampler.cpp:143-197).
"""
from __future__ import annotations

import argparse
import sys
import time
from typing import List, Optional


def parse_prompts(text: str) -> List[List[int]]:
    out = []
    for part in text.split(";"):
        ids = [int(x) for x in part.replace(",", " ").split()]
        if ids:
            out.append(ids)
    if not out:
        raise ValueError("the prompt holds no token ids")
    return out


def main(argv: Optional[List[str]] = None) -> int:
    from .config import EngineConfig

    ap = argparse.ArgumentParser(prog="generate", description=__doc__.split("\n\n")[0])
    ap.add_argument("model", nargs="?", default=None, help="folder with config.json and model.safetensors")
    ap.add_argument("prompt", nargs="?", default="1", help="token ids, e.g. \"5,17,3\"; ';' separates prompts")
    ap.add_argument("max_tokens", nargs="?", type=int, default=64)
    ap.add_argument("--random-config", default=None, metavar="CONFIG.json",
                    help="instead of a model folder: a config.json whose weights are drawn from --seed")
    ap.add_argument("--prompt-ids-file", default=None, help="file with one prompt (token ids) a line")
    ap.add_argument("--print-logits", type=int, default=0, metavar="N",
                    help="print the N largest logits at each prompt's last token")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--greedy", dest="greedy", action="store_true", default=True)
    ap.add_argument("--no-greedy", dest="greedy", action="store_false", help="draw from the distribution")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=0.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--page-size", type=int, default=EngineConfig().page_size)
    ap.add_argument("--max-cached-tokens", type=int, default=0, help="cache pool in tokens (0 = from free memory)")
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--kernels", choices=["fast", "plain"], default="fast")
    ap.add_argument("--ignore-eos", action="store_true")
    args = ap.parse_args(argv)

    from .engine.llm import LLM
    from .sampling import SamplingParams

    def log(msg: str) -> None:
        print(msg, file=sys.stderr, flush=True)

    if args.random_config is not None:
        # with --random-config the first two positionals are the prompt and max_tokens
        if args.model is not None:
            args.prompt, args.max_tokens = args.model, (int(args.prompt) if args.prompt != "1" else args.max_tokens)
        import json
        import tempfile

        from .config import config_from_dict
        from .weights import write_random_model
        with open(args.random_config, "r", encoding="utf-8") as f:
            config = config_from_dict(json.load(f))
        holder = tempfile.TemporaryDirectory(prefix="llmengine_b200_random_")
        args.model = write_random_model(config, args.seed, holder.name)
    elif args.model is None:
        ap.error("a model folder (or --random-config) is needed")
    if args.prompt_ids_file is not None:
        with open(args.prompt_ids_file, "r", encoding="utf-8") as f:
            prompts = parse_prompts(";".join(line.strip() for line in f if line.strip()))
    else:
        prompts = parse_prompts(args.prompt)
    log("[1/3] Loading model...")
    t0 = time.time()
    llm = LLM(args.model, dtype=args.dtype, page_size=args.page_size, max_cached_tokens=args.max_cached_tokens,
              max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
              prefill_chunk=args.prefill_chunk, kernels=args.kernels, seed=args.seed)
    log(f"      {time.time() - t0:.1f} s")
    sp = SamplingParams(greedy=args.greedy, top_k=args.top_k, top_p=args.top_p, temperature=args.temperature,
                        repetition_penalty=args.repetition_penalty, seed=args.seed)
    if args.print_logits > 0:
        from .engine.engine import StepEntry
        for i, p in enumerate(prompts):
            row = llm.engine.step([StepEntry(("logits", i), p, [len(p) - 1])], end=[("logits", i)])[0]
            top = row.topk(min(args.print_logits, row.numel()))
            print("logits " + " ".join(f"{int(t)}:{float(v):.6f}" for v, t in zip(top.values.tolist(), top.indices.tolist())))
    log(f"[2/3] Generating ({len(prompts)} prompt(s), up to {args.max_tokens} tokens each)...")
    t0 = time.time()
    outs = llm.generate(prompts, sp, args.max_tokens, eos_token_id=None if args.ignore_eos else "model")
    dt = time.time() - t0
    log("[3/3] Done")
    total = 0
    for o in outs:
        print(" ".join(str(t) for t in o.token_ids))
        total += len(o.token_ids)
    print(f"\n[Generated {total} tokens total]")
    log(f"      {total / max(dt, 1e-9):.1f} tokens/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
