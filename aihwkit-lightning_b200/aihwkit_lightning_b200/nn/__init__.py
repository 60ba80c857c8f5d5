"""Analog neural-network layers."""
from .modules import (
    AnalogBidirRNNLayer,
    AnalogContainerBase,
    AnalogConv1d,
    AnalogConv2d,
    AnalogConv3d,
    AnalogGRUCell,
    AnalogLayerBase,
    AnalogLinear,
    AnalogLSTMCell,
    AnalogLSTMCellCombinedWeight,
    AnalogReverseRNNLayer,
    AnalogRNN,
    AnalogRNNLayer,
    AnalogSequential,
    AnalogVanillaRNNCell,
    AnalogWrapper,
)
from .conversion import convert_to_analog, convert_to_digital

__all__ = ["AnalogConv1d", "AnalogConv2d", "AnalogConv3d", "AnalogLayerBase", "AnalogContainerBase", "AnalogLinear",
           "AnalogSequential", "AnalogWrapper", "AnalogRNN", "AnalogRNNLayer", "AnalogReverseRNNLayer",
           "AnalogBidirRNNLayer", "AnalogVanillaRNNCell", "AnalogLSTMCell", "AnalogLSTMCellCombinedWeight",
           "AnalogGRUCell", "convert_to_analog", "convert_to_digital"]
