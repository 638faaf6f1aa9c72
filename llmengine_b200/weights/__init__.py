"""Weights: the safetensors container, loading by tensor name, and the random-weights mode."""
from .loader import (WeightError, check_names_and_shapes, load_model_weights, random_model_weights, random_tensor,
                     stored_dtype, write_random_model)
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors

__all__ = ["SafetensorsError", "SafetensorsFile", "WeightError", "check_names_and_shapes", "load_model_weights",
           "open_model_files", "random_model_weights", "random_tensor", "stored_dtype", "write_random_model",
           "write_safetensors"]
