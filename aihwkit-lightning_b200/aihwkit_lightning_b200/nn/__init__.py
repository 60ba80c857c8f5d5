"""Analog neural-network layers."""
from .modules import AnalogConv2d, AnalogLayerBase, AnalogLinear
from .conversion import convert_to_analog, convert_to_digital

__all__ = ["AnalogConv2d", "AnalogLayerBase", "AnalogLinear", "convert_to_analog", "convert_to_digital"]
