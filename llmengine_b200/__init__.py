"""llmengine_b200: a single-GPU inference engine for B200 (sm_100a).

From a model folder (config.json + model.safetensors) to generated tokens: typed
configuration and architecture registry, weights by tensor name, layers put together from
parts, a paged cache with block tables, one step function for mixed batches, a scheduler,
samplers, and hand-written CUDA kernels.
"""
from .config import EngineConfig, load_config  # noqa: F401

__version__ = "0.1.0"
