"""Architectures assembled from parts.  Importing this package registers them."""
from .spec import ModelSpec, TensorBinding
from . import bifatar, llama, lobutar, rivetar, tolanex

__all__ = ["ModelSpec", "TensorBinding", "llama", "tolanex", "bifatar", "rivetar", "lobutar"]
