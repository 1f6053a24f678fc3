from . import dikusun, gefarax, qwen3, vibepel, zeridra  # noqa: F401  (register the architectures)
from .decoder import DecoderModel
from .loading import load_model, random_model

__all__ = ["DecoderModel", "load_model", "random_model"]
