"""``AnalogConv1d`` / ``AnalogConv2d`` / ``AnalogConv3d``: drop-ins for the reference layers
(`nn/modules/conv.py:123-360, 363-513, 516-677, 680-941`).

The convolution is evaluated as the analog linear operator on unfolded patches: the patch
axis is ordered (channel, kernel depth, kernel row, kernel column) like
``torch.nn.functional.unfold``, and analog tiles are cut along that axis, exactly as the
reference does.  2-D (and 1-D, which is 2-D with one row) patches come from the library's own
unfold kernel; 3-D patches are strided views of the padded input (PyTorch plumbing, off the
benchmarked path).
"""
from copy import deepcopy
from functools import reduce
from typing import Optional, Tuple, Union

import torch
from torch import Tensor
from torch.nn.modules.conv import _ConvNd
from torch.nn.modules.utils import _pair, _single, _triple

from ...simulator.configs import TorchInferenceRPUConfig
from ...simulator.enums import WeightClipType, WeightQuantizationType
from .. import functional as F
from .base import AnalogLayerBase
from .linear import _modified_weights


class _AnalogConvNd(AnalogLayerBase, _ConvNd):
    """Shared base of the analog convolutions."""

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
        out = F.analog_conv2d_rows(inp, self.weight.view(self.out_channels, -1), self.bias,
                                   self.input_range, self.input_range_update_idx, self.in_sizes,
                                   self.training, self.rpu_config, self.x_min, self.x_max,
                                   self.learnable_weight_clip, self.kernel_size, self.dilation, self.padding,
                                   self.stride)
        out_size = (im_shape[-2] + 2 * self.padding[0] - self.dilation[0] * (self.kernel_size[0] - 1) - 1
                    ) // self.stride[0] + 1
        if len(im_shape) == 3:
            return out.transpose(-1, -2).contiguous().view(self.out_channels, out_size, -1)
        out = out.view(im_shape[0], -1, self.out_channels).transpose(-1, -2).contiguous()
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


class AnalogConv1d(_AnalogConvNd):
    """1-D convolution on analog tiles; same signature as ``torch.nn.Conv1d`` plus ``rpu_config``.

    Held as a 2-D convolution over images of one row (`nn/modules/conv.py:394-436`): the weight
    parameter is ``[out, in, 1, k]`` and is squeezed to PyTorch's ``[out, in, k]`` in state dicts."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: Union[int, Tuple], stride=1,
                 padding=0, dilation=1, groups: int = 1, bias: bool = True, padding_mode: str = "zeros",
                 device=None, dtype=None, rpu_config: Optional[TorchInferenceRPUConfig] = None):
        kernel_size, stride = _single(kernel_size), _single(stride)
        padding, dilation = _single(padding), _single(dilation)
        if dilation != _single(1):
            raise ValueError("Only dilation = 1 is supported")
        super().__init__(in_channels, out_channels, (1, kernel_size[0]), (1, stride[0]), (0, padding[0]),
                         (1, dilation[0]), False, _pair(0), groups, bias, padding_mode, device, dtype,
                         rpu_config)
        self._register_load_state_dict_pre_hook(self._unsqueeze_loaded_weight)
        self._register_state_dict_hook(self._squeeze_saved_weight)

    def forward(self, inp: Tensor) -> Tensor:
        return super().forward(inp.unsqueeze(-2)).squeeze(-2)

    @classmethod
    def from_digital(cls, module: torch.nn.Conv1d, rpu_config: TorchInferenceRPUConfig) -> "AnalogConv1d":
        layer = cls(module.in_channels, module.out_channels, module.kernel_size, module.stride,
                    module.padding, module.dilation, module.groups, module.bias is not None,
                    module.padding_mode, device=module.weight.device, dtype=module.weight.dtype,
                    rpu_config=rpu_config)
        layer.set_weights_and_biases(module.weight.data.unsqueeze(-2),
                                     None if module.bias is None else module.bias.data)
        return layer

    @classmethod
    def to_digital(cls, module: "AnalogConv1d") -> torch.nn.Conv1d:
        digital = torch.nn.Conv1d(module.in_channels, module.out_channels, module.kernel_size[1],
                                  module.stride[1], module.padding[1], module.dilation[1], module.groups,
                                  module.bias is not None, module.padding_mode)
        digital.weight.data = module.weight.data.detach().clone().squeeze(-2)
        if module.bias is not None:
            digital.bias.data = module.bias.data.detach().clone()
        return digital.to(device=module.weight.device, dtype=module.weight.dtype)

    @staticmethod
    def _unsqueeze_loaded_weight(state_dict, prefix, *args, **kwargs):  # pylint: disable=unused-argument
        key = prefix + "weight"
        if key in state_dict and state_dict[key].ndim == 3:
            state_dict[key] = state_dict[key].unsqueeze(-2)

    @staticmethod
    def _squeeze_saved_weight(module, state_dict, prefix, local_metadata):  # pylint: disable=unused-argument
        key = prefix + "weight"
        if key in state_dict and state_dict[key].ndim == 4:
            state_dict[key] = state_dict[key].squeeze(-2)


def unfold3d(inp: Tensor, kernel_size, padding, stride) -> Tensor:
    """Patches of a ``[B, C, D, H, W]`` (or unbatched ``[C, D, H, W]``) volume as
    ``[B, patches, C * kD * kH * kW]``: rows are output positions (depth-major), the patch axis is
    ordered (channel, kernel depth, kernel row, kernel column) (`nn/modules/conv.py:42-104`,
    transposed here because the linear operator wants patches as rows)."""
    batched = inp.ndim == 5
    vol = inp if batched else inp.unsqueeze(0)
    vol = torch.nn.functional.pad(vol, (padding[2], padding[2], padding[1], padding[1], padding[0], padding[0]))
    views = vol.unfold(2, kernel_size[0], stride[0]).unfold(3, kernel_size[1], stride[1])
    views = views.unfold(4, kernel_size[2], stride[2])          # [B, C, nD, nH, nW, kD, kH, kW]
    views = views.permute(0, 2, 3, 4, 1, 5, 6, 7)               # [B, nD, nH, nW, C, kD, kH, kW]
    patches = views.reshape(views.shape[0], views.shape[1] * views.shape[2] * views.shape[3], -1)
    return patches if batched else patches.squeeze(0)


class AnalogConv3d(_AnalogConvNd):
    """3-D convolution on analog tiles; same signature as ``torch.nn.Conv3d`` plus ``rpu_config``
    (`nn/modules/conv.py:680-941`; dilation 1 only, like the reference)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: Union[int, Tuple], stride=1,
                 padding=0, dilation=1, groups: int = 1, bias: bool = True, padding_mode: str = "zeros",
                 device=None, dtype=None, rpu_config: Optional[TorchInferenceRPUConfig] = None):
        if _triple(dilation) != _triple(1):
            raise ValueError("Only dilation = 1 is supported")
        super().__init__(in_channels, out_channels, _triple(kernel_size), _triple(stride), _triple(padding),
                         _triple(dilation), False, _triple(0), groups, bias, padding_mode, device, dtype,
                         rpu_config)

    def forward(self, inp: Tensor) -> Tensor:
        self._check_forward_config()
        assert isinstance(self.padding, tuple), "Padding must be a tuple"
        patches = unfold3d(inp, self.kernel_size, self.padding, self.stride)
        out = F.analog_linear(patches, self.weight.view(self.out_channels, -1), self.bias,
                              self.input_range, self.input_range_update_idx, self.in_sizes,
                              self.training, self.rpu_config, self.x_min, self.x_max,
                              self.learnable_weight_clip)
        sizes = [(inp.shape[-3 + i] + 2 * self.padding[i] - (self.kernel_size[i] - 1) - 1) // self.stride[i] + 1
                 for i in range(3)]
        out = out.transpose(-1, -2).contiguous()
        if inp.ndim == 4:
            return out.view(self.out_channels, *sizes)
        return out.view(inp.shape[0], self.out_channels, *sizes)

    @classmethod
    def from_digital(cls, module: torch.nn.Conv3d, rpu_config: TorchInferenceRPUConfig) -> "AnalogConv3d":
        layer = cls(module.in_channels, module.out_channels, module.kernel_size, module.stride,
                    module.padding, module.dilation, module.groups, module.bias is not None,
                    module.padding_mode, device=module.weight.device, dtype=module.weight.dtype,
                    rpu_config=rpu_config)
        layer.set_weights_and_biases(module.weight.data, None if module.bias is None else module.bias.data)
        return layer

    @classmethod
    def to_digital(cls, module: "AnalogConv3d") -> torch.nn.Conv3d:
        digital = torch.nn.Conv3d(module.in_channels, module.out_channels, module.kernel_size,
                                  module.stride, module.padding, module.dilation, module.groups,
                                  module.bias is not None, module.padding_mode)
        digital.weight.data = module.weight.data.detach().clone()
        if module.bias is not None:
            digital.bias.data = module.bias.data.detach().clone()
        return digital.to(device=module.weight.device, dtype=module.weight.dtype)
