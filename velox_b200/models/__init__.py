from . import dobepel, qwen3  # register the architectures
from .decoder import DecoderModel

__all__ = ["DecoderModel", "dobepel", "qwen3"]
