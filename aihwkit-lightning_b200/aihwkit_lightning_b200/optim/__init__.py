"""Optimizers for analog layers."""
from .analog_optimizer import AnalogOptimizer

__all__ = ["AnalogOptimizer"]
