"""Random-weights mode as a command: writes a model folder from a configuration and a seed.

    python -m llmengine_b200.make_random_model CONFIG.json --seed S OUT_DIR [--dtype bfloat16|float32]

CONFIG.json holds the architecture's own config.json keys (`architectures` chooses the model).
OUT_DIR receives `config.json` and `model.safetensors`; every tensor is drawn from (seed, tensor
name) alone: matrices and the embedding ~ N(0, 0.02), norm gains ~ 1 + N(0, 0.1).  The reference
has no such mode (it loads GGUF files only: src/io/gguf_weight_loader.cpp); it exists so that the
file loader, the engine and the tests can run where no checkpoint can be had.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="make_random_model", description=__doc__.split("\n\n")[0])
    ap.add_argument("config", help="a config.json")
    ap.add_argument("out", help="folder to write config.json and model.safetensors into")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="type the tensors are stored in")
    ap.add_argument("--shard-bytes", type=int, default=0,
                    help="write several model-0000i-of-0000n.safetensors files of about this size each, with a "
                         "model.safetensors.index.json, as large checkpoints are laid out (0 = one file)")
    args = ap.parse_args(argv)

    from .config import ConfigError, config_from_dict
    from .weights import write_random_model

    try:
        with open(args.config, "r", encoding="utf-8") as f:
            config = config_from_dict(json.load(f))
    except (OSError, json.JSONDecodeError, ConfigError) as e:
        print(f"make_random_model: {e}", file=sys.stderr)
        return 2
    out = write_random_model(config, args.seed, args.out, dtype=args.dtype, shard_bytes=args.shard_bytes)
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
