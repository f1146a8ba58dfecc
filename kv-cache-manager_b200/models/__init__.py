"""Architectures assembled from parts.  Importing this package registers them."""
from .spec import ModelSpec, TensorBinding
from . import llama

__all__ = ["ModelSpec", "TensorBinding", "llama"]
