"""Zaverax model family: configuration reader and the CUDA-executed model class."""
from .config import LayerConfig, MixerConfig, ZaveraxConfig
from .model import Zaverax

__all__ = ["Zaverax", "ZaveraxConfig", "LayerConfig", "MixerConfig"]
