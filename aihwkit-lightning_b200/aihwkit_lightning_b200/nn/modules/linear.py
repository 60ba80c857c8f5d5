"""``AnalogLinear``: drop-in for the reference layer of the same name
(`nn/modules/linear.py:53-317`), computing through the sm_100a CUDA library."""
from copy import deepcopy
from typing import Optional, Tuple

import torch
from torch import Tensor
from torch.nn import Linear

from ...simulator.configs import TorchInferenceRPUConfig
from ...simulator.enums import WeightClipType, WeightQuantizationType
from .. import functional as F
from .base import AnalogLayerBase


class AnalogLinear(Linear, AnalogLayerBase):
    """Linear layer evaluated on (emulated) analog tiles: the input dimension is split into
    tiles of at most ``mapping.max_input_size`` rows; each tile has its own input range /
    DAC, weight noise, output noise and ADC, and the tile outputs are summed digitally."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None,
                 dtype=None, rpu_config: Optional[TorchInferenceRPUConfig] = None) -> None:
        if rpu_config is None:
            raise ValueError("rpu_config must be provided. Try TorchInferenceRPUConfig()")
        Linear.__init__(self, in_features, out_features, bias, device, dtype)
        self.rpu_config = rpu_config
        small_dev = "cpu" if str(device) == "meta" else device
        self.in_sizes = self.get_split_sizes(in_features, rpu_config.mapping.max_input_size)
        self.upper_end_of_slices = self._tile_upper_ends(small_dev)
        self.init_ir(init_value_ir=rpu_config.pre_post.input_range.init_value, init_value_counter=0,
                     device=small_dev, dtype=dtype)
        self.init_learnable_weight_ranges(self._tile_abs_max, device=small_dev, dtype=dtype)
        self.deprecation_adjustment()

    def _tile_abs_max(self) -> Tensor:
        w = self.weight.detach()
        if w.is_cuda:
            return F.sliced_abs_max(self.in_sizes, w)
        lo, rows = 0, []
        for size in self.in_sizes:  # construction-time only, before the module is on the GPU
            rows.append(w[:, lo:lo + size].abs().amax(dim=1))
            lo += size
        return torch.stack(rows)

    def forward(self, inp: Tensor) -> Tensor:  # pylint: disable=arguments-renamed
        self._check_forward_config()
        return F.analog_linear(inp, self.weight, self.bias, self.input_range,
                               self.input_range_update_idx, self.in_sizes, self.training,
                               self.rpu_config, self.x_min, self.x_max, self.learnable_weight_clip)

    @classmethod
    def from_digital(cls, module: Linear, rpu_config: TorchInferenceRPUConfig) -> "AnalogLinear":
        layer = cls(module.in_features, module.out_features, module.bias is not None,
                    device=module.weight.device, dtype=module.weight.dtype, rpu_config=rpu_config)
        layer.set_weights_and_biases(module.weight.data, None if module.bias is None else module.bias.data)
        return layer

    @classmethod
    def to_digital(cls, module: "AnalogLinear") -> Linear:
        digital = Linear(module.in_features, module.out_features, module.bias is not None)
        digital.weight.data = module.weight.data.detach().clone()
        if module.bias is not None:
            digital.bias.data = module.bias.data.detach().clone()
        return digital.to(device=module.weight.device, dtype=module.weight.dtype)

    @classmethod
    def move_to_meta(cls, module: Linear):
        module.to(device="meta")

    def set_weights(self, weight: Tensor) -> None:
        assert self.weight.shape == weight.shape, (
            f"weight shape mismatch. Got {weight.shape}, expected {self.weight.shape}")
        self.weight.data = weight.detach().clone()
        self.init_learnable_weight_ranges(self._tile_abs_max, device=weight.device, dtype=weight.dtype)

    def set_weights_and_biases(self, weight: Tensor, bias: Optional[Tensor] = None) -> None:
        self.set_weights(weight)
        if bias is not None:
            assert self.bias.shape == bias.shape, (
                f"bias shape mismatch. Got {bias.shape}, expected {self.bias.shape}")
            self.bias.data = bias.detach().clone()

    def get_weights_and_biases(self) -> Tuple[Tensor, Optional[Tensor]]:
        return (self.weight, self.bias)

    def clip_weights(self) -> None:
        """``W <- clamp(W, +-sigma*std(W))`` per tensor / per output channel; called by
        ``AnalogOptimizer`` after every step."""
        F.clip_weights_(self.weight, self.rpu_config.clip.type, self.rpu_config.clip.sigma)

    @torch.no_grad()
    def quantize_weights(self) -> None:
        """Bake the configured weight discretisation into ``weight`` and switch it off."""
        if (self.rpu_config.modifier.quantization_type != WeightQuantizationType.NONE
                or self.rpu_config.clip.type == WeightClipType.LEARNABLE_PER_CHANNEL):
            self.weight.data = _modified_weights(self, self.weight.data)
        AnalogLayerBase.quantize_weights(self)

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


def _modified_weights(layer, weight2d: Tensor) -> Tensor:
    """Discretised copy of a 2-D CUDA weight, produced by the forward's weight pre-pass."""
    from ...simulator.configs import TorchInferenceRPUConfig as Cfg

    cfg = Cfg()
    cfg.modifier.quantization_type = layer.rpu_config.modifier.quantization_type
    cfg.modifier.res = layer.rpu_config.modifier.res
    cfg.mapping.max_input_size = layer.rpu_config.mapping.max_input_size
    lwc = None
    if layer.rpu_config.clip.type == WeightClipType.LEARNABLE_PER_CHANNEL:
        cfg.clip.type = WeightClipType.LEARNABLE_PER_CHANNEL
        lwc = layer.learnable_weight_clip
    capture: dict = {}
    probe = torch.zeros(1, weight2d.shape[1], device=weight2d.device, dtype=weight2d.dtype)
    with F.operator_settings(capture=capture):
        F.analog_linear(probe, weight2d, None, None, None, layer.in_sizes, False, cfg, None, None, lwc)
    return capture["w_mod"].clone()
