"""``AnalogConv2d``: drop-in for the reference layer (`nn/modules/conv.py:123-360,516-677`).

The convolution is evaluated as the analog linear operator on unfolded patches: the patch
axis is ordered (channel, kernel row, kernel column) like ``torch.nn.functional.unfold``, and
analog tiles are cut along that axis, exactly as the reference does.
"""
from copy import deepcopy
from functools import reduce
from typing import Optional, Tuple, Union

import torch
from torch import Tensor
from torch.nn.modules.conv import _ConvNd
from torch.nn.modules.utils import _pair

from ...simulator.configs import TorchInferenceRPUConfig
from ...simulator.enums import WeightClipType, WeightQuantizationType
from .. import functional as F
from .base import AnalogLayerBase
from .linear import _modified_weights


class _AnalogConvNd(AnalogLayerBase, _ConvNd):
    """Shared base of the analog convolutions (only 2-D is provided)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, transposed,
                 output_padding, groups, bias, padding_mode, device=None, dtype=None,
                 rpu_config: Optional[TorchInferenceRPUConfig] = None):
        if groups != 1:
            raise ValueError("Only one group is supported")
        if padding_mode != "zeros":
            raise ValueError('Only "zeros" padding mode is supported')
        assert rpu_config is not None, "RPU config must be provided"
        _ConvNd.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation,
                         transposed, output_padding, groups, bias, padding_mode, device, dtype)
        small_dev = "cpu" if str(device) == "meta" else device
        self.in_features = self.get_tile_size(in_channels, groups, kernel_size)
        self.out_features = out_channels
        self.rpu_config = rpu_config
        self.in_sizes = self.get_split_sizes(self.in_features, rpu_config.mapping.max_input_size)
        self.upper_end_of_slices = self._tile_upper_ends(small_dev)
        self.init_ir(init_value_ir=rpu_config.pre_post.input_range.init_value, init_value_counter=0,
                     device=small_dev, dtype=dtype)
        self.init_learnable_weight_ranges(self._tile_abs_max, device=small_dev, dtype=dtype)
        self.deprecation_adjustment()

    def _tile_abs_max(self) -> Tensor:
        w = self.weight.detach().reshape(self.out_channels, -1)
        if w.is_cuda:
            return F.sliced_abs_max(self.in_sizes, w)
        lo, rows = 0, []
        for size in self.in_sizes:
            rows.append(w[:, lo:lo + size].abs().amax(dim=1))
            lo += size
        return torch.stack(rows)

    def get_tile_size(self, in_channels: int, groups: int, kernel_size: Tuple[int, ...]) -> int:
        return (in_channels // groups) * reduce(lambda a, b: a * b, kernel_size)

    @classmethod
    def move_to_meta(cls, module: _ConvNd):
        module.to(device="meta")

    def set_weights(self, weight: Tensor) -> None:
        assert self.weight.shape == weight.shape, (
            f"weight shape mismatch. Got {weight.shape}, expected {self.weight.shape}")
        self.weight.data = weight.detach().clone()

    def set_weights_and_biases(self, weight: Tensor, bias: Optional[Tensor] = None) -> None:
        self.set_weights(weight)
        if bias is not None:
            assert self.bias is not None and self.bias.shape == bias.shape, "bias shape mismatch"
            self.bias.data = bias.detach().clone()

    def get_weights_and_biases(self) -> Tuple[Tensor, Optional[Tensor]]:
        return (self.weight, self.bias)

    def clip_weights(self) -> None:
        F.clip_weights_(self.weight, self.rpu_config.clip.type, self.rpu_config.clip.sigma)

    @torch.no_grad()
    def quantize_weights(self) -> None:
        if (self.rpu_config.modifier.quantization_type != WeightQuantizationType.NONE
                or self.rpu_config.clip.type == WeightClipType.LEARNABLE_PER_CHANNEL):
            w2d = self.weight.data.reshape(self.out_channels, -1).contiguous()
            self.weight.data = _modified_weights(self, w2d).view_as(self.weight)
        AnalogLayerBase.quantize_weights(self)

    def forward(self, inp: Tensor) -> Tensor:
        self._check_forward_config()
        im_shape = inp.shape
        assert isinstance(self.padding, tuple), "Padding must be a tuple"
        patches = F.unfold2d(inp, self.kernel_size, self.dilation, self.padding, self.stride)
        out = F.analog_linear(patches, self.weight.view(self.out_channels, -1), self.bias,
                              self.input_range, self.input_range_update_idx, self.in_sizes,
                              self.training, self.rpu_config, self.x_min, self.x_max,
                              self.learnable_weight_clip)
        out = out.transpose(-1, -2).contiguous()
        out_size = (im_shape[-2] + 2 * self.padding[0] - self.dilation[0] * (self.kernel_size[0] - 1) - 1
                    ) // self.stride[0] + 1
        if len(im_shape) == 3:
            return out.view(self.out_channels, out_size, -1)
        return out.view(im_shape[0], self.out_channels, out_size, -1)

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        super()._save_to_state_dict(destination, prefix, keep_vars)
        # pylint: disable=protected-access
        destination._metadata[prefix.split(".")[0]]["rpu_config"] = deepcopy(self.rpu_config)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)
        if "rpu_config" in local_metadata:
            self.rpu_config = deepcopy(local_metadata["rpu_config"])


class AnalogConv2d(_AnalogConvNd):
    """2-D convolution on analog tiles; same signature as ``torch.nn.Conv2d`` plus ``rpu_config``."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: Union[int, Tuple], stride=1,
                 padding=0, dilation=1, groups: int = 1, bias: bool = True, padding_mode: str = "zeros",
                 device=None, dtype=None, rpu_config: Optional[TorchInferenceRPUConfig] = None):
        super().__init__(in_channels, out_channels, _pair(kernel_size), _pair(stride), _pair(padding),
                         _pair(dilation), False, _pair(0), groups, bias, padding_mode, device, dtype,
                         rpu_config)

    @classmethod
    def from_digital(cls, module: torch.nn.Conv2d, rpu_config: TorchInferenceRPUConfig) -> "AnalogConv2d":
        layer = cls(module.in_channels, module.out_channels, module.kernel_size, module.stride,
                    module.padding, module.dilation, module.groups, module.bias is not None,
                    module.padding_mode, device=module.weight.device, dtype=module.weight.dtype,
                    rpu_config=rpu_config)
        layer.set_weights_and_biases(module.weight.data, None if module.bias is None else module.bias.data)
        return layer

    @classmethod
    def to_digital(cls, module: "AnalogConv2d") -> torch.nn.Conv2d:
        digital = torch.nn.Conv2d(module.in_channels, module.out_channels, module.kernel_size,
                                  module.stride, module.padding, module.dilation, module.groups,
                                  module.bias is not None, module.padding_mode)
        digital.weight.data = module.weight.data.detach().clone()
        if module.bias is not None:
            digital.bias.data = module.bias.data.detach().clone()
        return digital.to(device=module.weight.device, dtype=module.weight.dtype)
