"""Analog layer modules."""
from .base import AnalogLayerBase, split_sizes
from .conv import AnalogConv2d
from .linear import AnalogLinear

__all__ = ["AnalogLayerBase", "AnalogConv2d", "AnalogLinear", "split_sizes"]
