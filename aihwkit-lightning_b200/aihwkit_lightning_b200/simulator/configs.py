"""RPU configuration dataclasses.

Field names, defaults and nesting follow the reference one to one
(`simulator/configs/configs.py:27-88`, `simulator/parameters/io.py:23-59`,
`inference.py:30-90`, `mapping.py:22-38`, `pre_post.py:23-98`): they are plain data read by
the layer on every call and flattened into the ``AlDesc`` struct of the CUDA library.
"""
from dataclasses import dataclass, field, fields

from .enums import (
    WeightClipType,
    WeightModifierType,
    WeightNoiseInjectionType,
    WeightQuantizationType,
)


class _Printable:
    """``str()`` that lists one field per line when there are more than three."""

    def __str__(self) -> str:
        parts = []
        for item in fields(self):  # type: ignore[arg-type]
            text = str(getattr(self, item.name))
            parts.append(f"{item.name}={text}")
        name = type(self).__name__
        if len(parts) > 3 or any("\n" in p for p in parts):
            body = ",\n".join(parts)
            body = "\n".join("    " + line for line in body.split("\n"))
            return f"{name}(\n{body}\n)"
        return f"{name}({', '.join(parts)})"


@dataclass
class IOParameters(_Printable):
    """Periphery of the analog matrix-vector product."""

    inp_res: float = -1
    """DAC steps (``254``) or resolution (``1/254``); ``<= 0`` switches the DAC off."""
    out_noise: float = 0.0
    """Std-dev of the Gaussian noise added to every tile output during training."""
    out_noise_per_channel: bool = False
    """Scale the output noise by each channel's abs-max instead of the tile's."""
    out_bound: float = 0.0
    """ADC bound in units of ``input_range * abs-max``; ``<= 0`` means no clipping."""
    out_res: float = -1
    """ADC steps or resolution; ``<= 0`` switches the ADC quantisation off."""


@dataclass
class WeightModifierParameter(_Printable):
    """Weight noise / discretisation applied in the forward pass."""

    std_dev: float = 0.0
    res: float = 0.0
    enable_during_test: bool = False
    type: WeightModifierType = field(default_factory=lambda: WeightModifierType.NONE)
    noise_type: WeightNoiseInjectionType = field(
        default_factory=lambda: WeightNoiseInjectionType.NONE
    )
    quantization_type: WeightQuantizationType = field(
        default_factory=lambda: WeightQuantizationType.NONE
    )


@dataclass
class WeightClipParameter(_Printable):
    """Weight clipping after the optimizer step."""

    sigma: float = -1.0
    type: WeightClipType = field(default_factory=lambda: WeightClipType.NONE)


@dataclass
class MappingParameter(_Printable):
    """How the logical weight matrix maps to analog tiles."""

    max_input_size: int = -1
    """Rows of one analog tile; the input dimension is split evenly into
    ``ceil(in_features / max_input_size)`` tiles.  ``<= 0``: a single tile."""


@dataclass
class InputRangeParameter(_Printable):
    """Input range (DAC clipping range) handling."""

    fast_mode: bool = False
    act_range_momentum: float = 0.95
    enable: bool = False
    dynamic: bool = False
    learn_input_range: bool = True
    init_value: float = 3.0
    init_from_data: int = 100
    init_std_alpha: float = 3.0
    decay: float = 0.001
    input_min_percentage: float = 0.95


@dataclass
class PrePostProcessingParameter(_Printable):
    """Digital pre/post processing around the tiles."""

    input_range: InputRangeParameter = field(default_factory=InputRangeParameter)


@dataclass
class TorchInferenceRPUConfig:
    """Configuration of an analog layer used for hardware-aware training and inference."""

    forward: IOParameters = field(default_factory=IOParameters)
    clip: WeightClipParameter = field(default_factory=WeightClipParameter)
    modifier: WeightModifierParameter = field(default_factory=WeightModifierParameter)
    mapping: MappingParameter = field(default_factory=MappingParameter)
    pre_post: PrePostProcessingParameter = field(default_factory=PrePostProcessingParameter)
