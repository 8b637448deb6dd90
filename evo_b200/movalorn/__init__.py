"""Movalorn model family: configuration reader and the CUDA-executed model class."""
from .config import LayerConfig, MixerConfig, MlpConfig, MovalornConfig
from .model import Movalorn

__all__ = ["Movalorn", "MovalornConfig", "LayerConfig", "MixerConfig", "MlpConfig"]
