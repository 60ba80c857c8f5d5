"""Mixin shared by the analog layers: layer iteration, input-range state, config upgrades.

State layout (names, shapes, dtypes) equals the reference's (`nn/modules/base.py:104-159`), so
checkpoints move between the two implementations unchanged:

* ``input_range``             Parameter ``[n_tiles]`` (only for a learned / fixed range)
* ``input_range_update_idx``  buffer ``[n_tiles]``, counts init-from-data updates
* ``x_min`` / ``x_max``       buffers ``[n_tiles]`` (fast mode of the reference)
* ``learnable_weight_clip``   Parameter ``[n_tiles, out]`` (only for LEARNABLE_PER_CHANNEL)
"""
import warnings
from typing import Callable, Generator, List, Tuple

import torch
from torch import Tensor
from torch.nn import Parameter

from ...simulator.enums import (
    WeightClipType,
    WeightModifierType,
    WeightNoiseInjectionType,
    WeightQuantizationType,
)


def split_sizes(size: int, split_max_size: int) -> List[int]:
    """Widths of the analog tiles along the input dimension: ``ceil(size/max)`` tiles as equal
    as possible, the first ``size % n`` one wider (`nn/modules/linear.py:155-170`)."""
    if split_max_size <= 0:
        return [size]
    n_tiles = -(-size // split_max_size)
    base, extra = divmod(size, n_tiles)
    return [base + 1] * extra + [base] * (n_tiles - extra)


class AnalogLayerBase:
    """Functionality every analog layer has."""

    IS_CONTAINER: bool = False

    def named_analog_layers(self) -> Generator[Tuple[str, "AnalogLayerBase"], None, None]:
        """(name, layer) for every analog leaf layer below (and including) this module."""
        for name, module in self.named_modules():  # type: ignore[attr-defined]
            if isinstance(module, AnalogLayerBase) and not module.IS_CONTAINER:
                yield name, module

    def analog_layers(self) -> Generator["AnalogLayerBase", None, None]:
        for _, module in self.named_analog_layers():
            yield module

    def apply_to_analog_layers(self, fn: Callable) -> "AnalogLayerBase":
        for module in self.analog_layers():
            fn(module)
        return self

    @classmethod
    def move_to_meta(cls, _):
        return

    def clip_weights(self) -> None:
        return

    def get_split_sizes(self, size: int, split_max_size: int) -> List[int]:
        return split_sizes(size, split_max_size)

    # -- state ---------------------------------------------------------------------------
    def init_learnable_weight_ranges(self, init_value, device, dtype) -> None:
        """``init_value`` may be a tensor or a callable returning one (only evaluated when the
        learnable clip is configured)."""
        # pylint: disable=attribute-defined-outside-init
        if self.rpu_config.clip.type == WeightClipType.LEARNABLE_PER_CHANNEL:
            value = init_value() if callable(init_value) else init_value
            self.learnable_weight_clip = Parameter(value.to(dtype=dtype, device=device), requires_grad=True)
        else:
            self.learnable_weight_clip = None

    def init_ir(self, device, dtype, init_value_ir: float, init_value_counter: int = 0) -> None:
        # pylint: disable=attribute-defined-outside-init
        cfg = self.rpu_config.pre_post.input_range
        n_tiles = len(self.in_sizes)
        if cfg.enable and not cfg.dynamic:
            self.input_range = Parameter(
                torch.full((n_tiles,), float(init_value_ir), dtype=dtype, device=device),
                requires_grad=cfg.learn_input_range,
            )
            self.register_buffer(
                "input_range_update_idx",
                torch.full((n_tiles,), float(init_value_counter), dtype=dtype, device=device),
            )
            self.register_buffer("x_min", torch.zeros(n_tiles, dtype=dtype, device=device) - 1e-5)
            self.register_buffer("x_max", torch.zeros(n_tiles, dtype=dtype, device=device) + 1e-5)
        else:
            self.input_range = None
            self.input_range_update_idx = None
            self.x_min = None
            self.x_max = None

    def deprecation_adjustment(self) -> None:
        """Translate the pre-v2 ``modifier.type`` into ``noise_type`` / ``quantization_type``
        (`nn/modules/base.py:161-206`)."""
        mod = self.rpu_config.modifier
        old = mod.type
        if old != WeightModifierType.NONE:
            warnings.warn(
                "You are using the deprecated rpu_config.modifier.type. This model was likely "
                "trained with AIHWKIT-Lightning version <2."
            )
            name = old.name
            if name.endswith("ADD_NORMAL_PER_CHANNEL"):
                mod.noise_type = WeightNoiseInjectionType.ADD_NORMAL_PER_CHANNEL
            elif name.endswith("ADD_NORMAL"):
                mod.noise_type = WeightNoiseInjectionType.ADD_NORMAL
            else:
                mod.noise_type = WeightNoiseInjectionType.NONE
            if name in ("DISCRETIZE", "DISCRETIZE_ADD_NORMAL"):
                mod.quantization_type = WeightQuantizationType.DISCRETIZE
            elif name in ("DISCRETIZE_PER_CHANNEL", "DISCRETIZE_ADD_NORMAL_PER_CHANNEL"):
                mod.quantization_type = WeightQuantizationType.DISCRETIZE_PER_CHANNEL
            else:
                mod.quantization_type = WeightQuantizationType.NONE
        if mod.enable_during_test:
            mod.enable_during_test = False
            warnings.warn(
                "You created a modifier with enable_during_test set True. "
                "This is deprecated and was set to False."
            )

    def quantize_weights(self) -> None:
        warnings.warn("Modified the rpu_config because quantize_weights was called.")
        self.rpu_config.modifier.quantization_type = WeightQuantizationType.NONE
        self.rpu_config.clip.type = WeightClipType.NONE

    # -- helpers shared by linear and conv ---------------------------------------------------
    def _check_forward_config(self) -> None:
        fwd = self.rpu_config.forward
        if fwd.out_res > 0:
            assert fwd.out_bound > 0, "Out quant. without a bound."
            assert self.rpu_config.pre_post.input_range.enable, "Out quant. without IR."
        if self.rpu_config.clip.type == WeightClipType.LEARNABLE_PER_CHANNEL:
            assert self.learnable_weight_clip is not None, "Learnable weight clipping tensor not initialized."

    def _tile_upper_ends(self, device) -> Tensor:
        return torch.tensor(self.in_sizes, device=device).cumsum(dim=0, dtype=torch.int32).contiguous()
