"""Architectures of this engine. Importing the package registers them."""
from . import qwen2
from .loading import build_model, load_model, load_random_model, write_random_model

__all__ = ["qwen2", "build_model", "load_model", "load_random_model", "write_random_model"]
