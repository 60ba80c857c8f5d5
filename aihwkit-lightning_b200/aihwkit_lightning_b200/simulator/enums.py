"""Enumerations of the RPU configuration.

Member names and string values equal the reference's (`simulator/parameters/enums.py:22-90`):
they end up in pickled checkpoints (`_metadata["rpu_config"]`), so they are part of the
drop-in contract.
"""
from enum import Enum


class WeightModifierType(Enum):
    """Pre-v2 combined modifier switch; only read by ``deprecation_adjustment``."""

    NONE = "None"
    DISCRETIZE = "Discretize"
    DISCRETIZE_PER_CHANNEL = "DiscretizePerChannel"
    ADD_NORMAL = "AddNormal"
    ADD_NORMAL_PER_CHANNEL = "AddNormalPerChannel"
    DISCRETIZE_ADD_NORMAL = "DiscretizeAddNormal"
    DISCRETIZE_ADD_NORMAL_PER_CHANNEL = "DiscretizeAddNormalPerChannel"


class WeightNoiseInjectionType(Enum):
    """Additive Gaussian weight noise during training: off, scaled by the tile's abs-max, or
    scaled by each output channel's abs-max inside the tile."""

    NONE = "None"
    ADD_NORMAL = "AddNormal"
    ADD_NORMAL_PER_CHANNEL = "AddNormalPerChannel"


class WeightQuantizationType(Enum):
    """On-the-fly weight discretisation: off, one step per tile, or one step per channel."""

    NONE = "None"
    DISCRETIZE = "Discretize"
    DISCRETIZE_PER_CHANNEL = "DiscretizePerChannel"


class WeightClipType(Enum):
    """Weight clipping applied after each optimizer step (Gaussian variants) or learned."""

    NONE = "None"
    LAYER_GAUSSIAN = "LayerGaussian"
    LAYER_GAUSSIAN_PER_CHANNEL = "LayerGaussianPerChannel"
    LEARNABLE_PER_CHANNEL = "LearnablePerChannel"
