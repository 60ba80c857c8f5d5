"""Analog neural-network layers."""
from .modules import AnalogConv1d, AnalogConv2d, AnalogConv3d, AnalogLayerBase, AnalogLinear
from .conversion import convert_to_analog, convert_to_digital

__all__ = ["AnalogConv1d", "AnalogConv2d", "AnalogConv3d", "AnalogLayerBase", "AnalogLinear", "convert_to_analog",
           "convert_to_digital"]
