"""Weights: safetensors container I/O, loading by tensor name, random-weights mode."""
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors
from .loader import WeightError, load_from_tensors, load_weights, target_dtype
from .random_init import random_tensors, write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "open_model_files", "write_safetensors",
           "WeightError", "load_from_tensors", "load_weights", "target_dtype", "random_tensors",
           "write_random_model"]
