"""Analog layer modules."""
from .base import AnalogLayerBase, split_sizes
from .conv import AnalogConv1d, AnalogConv2d, AnalogConv3d
from .linear import AnalogLinear

__all__ = ["AnalogLayerBase", "AnalogConv1d", "AnalogConv2d", "AnalogConv3d", "AnalogLinear", "split_sizes"]
