"""Configuration: the typed model configuration, the registry from an
architecture's name to its configuration class, and the engine's own options."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Type

from .qwen3 import ConfigError, Qwen3Config
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec


@dataclass(frozen=True)
class Architecture:
    """What the engine needs to know about one architecture: how to read its
    config.json, and (through the configuration's `model_spec()`) its layers."""

    name: str
    config_class: Any

    def read_config(self, d: Mapping[str, Any]):
        return self.config_class.from_dict(d)


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any) -> None:
    """Register an architecture under the name that config.json gives in
    `architectures[0]`.  `config_class` needs `from_dict(dict)`, `model_spec()`,
    `to_dict()` and `canonical_tensor_name(name)`."""
    if name in ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    ARCHITECTURES[name] = Architecture(name, config_class)


def find_architecture(name: str) -> Architecture:
    try:
        return ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(sorted(ARCHITECTURES)) or '(none)'}") from None


def config_from_dict(d: Mapping[str, Any]):
    archs = d.get("architectures")
    if not archs:
        raise ConfigError("config.json lacks required key(s): architectures")
    return find_architecture(str(archs[0])).read_config(d)


def load_config(model_dir: str):
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path} does not exist") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    return config_from_dict(d)


register_architecture(Qwen3Config.ARCHITECTURE, Qwen3Config)


@dataclass
class EngineConfig:
    """Options of the engine itself (none of them is a property of the model).

    The reference hard-codes these in its examples (page size 16 and 256 pages in
    examples/generate_paged.cpp:173-174, at most 4 requests in
    include/minillm/runtime/continuous_batch_scheduler.h:43-45).  Pages here hold 64 tokens by
    default: a page of one head is then one 8 KB or 16 KB TMA box, and the tensor-core attention
    over a prompt measured 62.7 us per layer against 64.9 us with pages of 16 (2,048 tokens, 32 query
    and 8 key/value heads of 128); every power of two from 8 to 128 is served by the same kernels.
    """

    dtype: str = "bfloat16"              # "bfloat16" or "float32"
    page_size: int = 64                  # tokens per cache page
    max_cached_tokens: int = 0           # cache pool size in tokens; 0 = from free device memory
    gpu_memory_fraction: float = 0.85    # share of free memory the pool may take when sized automatically
    max_num_seqs: int = 64               # requests alive at once (also the number of state slots)
    max_num_batched_tokens: int = 2048   # token budget of one step
    prefill_chunk: int = 2048            # longest prompt portion of one request in one step
    max_model_len: int = 0               # 0 = the model's max_position_embeddings
    seed: int = 42                       # default sampling seed, as the reference's Sampler(42)
    use_cuda_graphs: bool = True         # capture decode-only steps
    # which kernels serve the operations: "fast", "plain" (the plain twins and the library product everywhere), or a
    # mapping operation -> variant that exchanges single kernels inside the whole model, e.g.
    # {"attention.portion": "mma", "linear": "cublas"} (the operations and their variants: executor.h)
    kernels: Any = "fast"
    device: str = "cuda:0"

    def __post_init__(self) -> None:
        if self.dtype in ("bf16",):
            self.dtype = "bfloat16"
        if self.dtype in ("fp32", "f32"):
            self.dtype = "float32"
        if self.dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        if self.page_size <= 0 or self.page_size > 256:
            raise ConfigError(f"page_size must be in 1..256, got {self.page_size}")
        if not (self.kernels in ("fast", "plain") or isinstance(self.kernels, Mapping)):
            raise ConfigError(f"kernels must be 'fast', 'plain' or a mapping operation -> variant, got {self.kernels!r}")
        for k in ("max_num_seqs", "max_num_batched_tokens", "prefill_chunk"):
            if getattr(self, k) <= 0:
                raise ConfigError(f"{k} must be positive")


__all__ = [
    "ARCHITECTURES", "Architecture", "ConfigError", "EngineConfig", "LayerRun", "LayerSpec", "ModelSpec",
    "PartSpec", "Qwen3Config", "config_from_dict", "find_architecture", "load_config", "register_architecture",
]
