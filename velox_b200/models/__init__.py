from . import buvuzen, dobepel, qwen3  # register the architectures
from .decoder import DecoderModel

__all__ = ["DecoderModel", "buvuzen", "dobepel", "qwen3"]
