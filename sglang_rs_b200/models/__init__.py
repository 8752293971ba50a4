"""Architectures.  Importing this package registers every one of them."""
from . import qwen3  # noqa: F401
from .decoder import DecoderModel, LayerCall

__all__ = ["DecoderModel", "LayerCall"]
