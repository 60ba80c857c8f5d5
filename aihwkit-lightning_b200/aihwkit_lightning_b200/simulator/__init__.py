"""Configuration objects of the analog layers."""
from .enums import (
    WeightClipType,
    WeightModifierType,
    WeightNoiseInjectionType,
    WeightQuantizationType,
)
from .configs import (
    InputRangeParameter,
    IOParameters,
    MappingParameter,
    PrePostProcessingParameter,
    TorchInferenceRPUConfig,
    WeightClipParameter,
    WeightModifierParameter,
)

__all__ = [
    "WeightClipType",
    "WeightModifierType",
    "WeightNoiseInjectionType",
    "WeightQuantizationType",
    "InputRangeParameter",
    "IOParameters",
    "MappingParameter",
    "PrePostProcessingParameter",
    "TorchInferenceRPUConfig",
    "WeightClipParameter",
    "WeightModifierParameter",
]
