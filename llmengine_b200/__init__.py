"""llmengine_b200: a single-GPU inference engine for B200 (sm_100a).

From a model folder (config.json + model.safetensors) to generated tokens: typed
configuration and architecture registry, weights by tensor name, layers put together from
parts, a paged cache with block tables, one step function for mixed batches, a scheduler,
samplers, and hand-written CUDA kernels.
"""
from .config import EngineConfig, load_config  # noqa: F401
from .sampling import SamplingParams  # noqa: F401


def __getattr__(name):
    # the engine classes import torch-heavy modules: resolve them on first use
    if name in ("LLM", "GenerationOutput"):
        from .engine import llm
        return getattr(llm, name)
    if name in ("Engine", "StepEntry", "StepError"):
        from .engine import engine
        return getattr(engine, name)
    raise AttributeError(name)

__version__ = "0.1.0"
