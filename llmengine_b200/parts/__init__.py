"""The parts a layer is put together from.  Importing this package registers the built-in kinds."""
from .base import (PagedKVSpec, Part, Runtime, StateSpec, WeightSpec, build_part, register_part, registered,
                   unregister_part)
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (registration)

__all__ = ["PagedKVSpec", "Part", "Runtime", "StateSpec", "WeightSpec", "build_part", "register_part",
           "registered", "unregister_part"]
