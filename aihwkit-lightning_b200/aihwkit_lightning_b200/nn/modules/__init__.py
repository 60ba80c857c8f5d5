"""Analog layer modules."""
from .base import AnalogLayerBase, split_sizes
from .container import AnalogContainerBase, AnalogSequential, AnalogWrapper
from .conv import AnalogConv1d, AnalogConv2d, AnalogConv3d
from .linear import AnalogLinear
from .rnn import (
    AnalogBidirRNNLayer,
    AnalogGRUCell,
    AnalogLSTMCell,
    AnalogLSTMCellCombinedWeight,
    AnalogReverseRNNLayer,
    AnalogRNN,
    AnalogRNNLayer,
    AnalogVanillaRNNCell,
    LSTMState,
    ModularRNN,
)

__all__ = ["AnalogLayerBase", "AnalogContainerBase", "AnalogSequential", "AnalogWrapper", "AnalogConv1d",
           "AnalogConv2d", "AnalogConv3d", "AnalogLinear", "AnalogRNN", "AnalogRNNLayer", "AnalogReverseRNNLayer",
           "AnalogBidirRNNLayer", "AnalogVanillaRNNCell", "AnalogLSTMCell", "AnalogLSTMCellCombinedWeight",
           "AnalogGRUCell", "LSTMState", "ModularRNN", "split_sizes"]
