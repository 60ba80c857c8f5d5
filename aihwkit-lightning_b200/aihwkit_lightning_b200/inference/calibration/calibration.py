"""Post-training calibration of the DAC input ranges (`inference/calibration/calibration.py:35-320`).

A model whose layers run without an input range is fed calibration batches; forward pre-hooks on
its analog layers collect per-tile statistics of the layer inputs (for convolutions: of the
unfolded patches) and the ranges derived from them are installed as the layers' static
``input_range``.  The statistics are the per-tile reductions of the forward path, evaluated on
the device by the library's own kernels (abs-max, unbiased std) or, for quantiles, by
``torch.quantile``; nothing is copied to the host per batch except the cached samples of
``CACHE_QUANTILE``.
"""
from copy import deepcopy
from enum import Enum
from typing import Dict, Iterable, List, Optional, Tuple

import torch
from torch import Tensor
from torch.nn import Module, Parameter

from ...exceptions import ConfigError
from ...nn import functional as F
from ...nn.modules.base import AnalogLayerBase
from ...nn.modules.conv import AnalogConv1d, AnalogConv3d, _AnalogConvNd, unfold3d
from ...simulator.enums import WeightNoiseInjectionType


class InputRangeCalibrationType(Enum):
    """How the ranges are derived from the calibration inputs."""

    NONE = "None"
    MOVING_STD = "MovingStd"            # running mean over batches of init_std_alpha * std(tile inputs)
    MOVING_QUANTILE = "MovingQuantile"  # running mean over batches of the tile's quantile
    CACHE_QUANTILE = "CacheQuantile"    # quantile over a cache of up to max_samples input rows
    MAX = "Max"                         # abs-max over everything seen


def _named_analog_layers(model: Module) -> List[Tuple[str, AnalogLayerBase]]:
    return [(name, mod) for name, mod in model.named_modules()
            if isinstance(mod, AnalogLayerBase) and not mod.IS_CONTAINER]


def _layer_rows(mod: AnalogLayerBase, x: Tensor) -> Tensor:
    """The layer's input as the rows its tiles see, all-zero rows dropped."""
    if isinstance(mod, AnalogConv3d):
        x = unfold3d(x, mod.kernel_size, mod.padding, mod.stride)
    elif isinstance(mod, _AnalogConvNd):
        if isinstance(mod, AnalogConv1d):
            x = x.unsqueeze(-2)  # held as a 2-D convolution over images of one row
        x = F.unfold2d(x, mod.kernel_size, mod.dilation, mod.padding, mod.stride)
    rows = x.reshape(-1, x.shape[-1])
    return rows[~(rows == 0.0).all(-1)].contiguous()


def _tile_slices(in_sizes: List[int]):
    lo = 0
    for t, size in enumerate(in_sizes):
        yield t, lo, lo + size
        lo += size


class _Collector:
    """Forward pre-hook of one layer."""

    def __init__(self, mod: AnalogLayerBase, kind: InputRangeCalibrationType, quantile: float, max_samples: int):
        self.mod, self.kind, self.quantile, self.max_samples = mod, kind, quantile, max_samples
        self.cache: Optional[Tensor] = None   # CACHE_QUANTILE: rows on the host; MAX: [T] on the device

    def __call__(self, mod, args, kwargs):
        x = args[0] if args else kwargs["inp"]
        rows = _layer_rows(mod, x.detach())
        if rows.shape[0] == 0:
            return
        kind = self.kind
        if kind == InputRangeCalibrationType.CACHE_QUANTILE:
            new = rows.float().cpu()
            cache = new if self.cache is None else torch.cat([self.cache, new])
            self.cache = cache[torch.randperm(cache.shape[0])[: self.max_samples]]
        elif kind == InputRangeCalibrationType.MAX:
            tile_max = F.sliced_abs_max(mod.in_sizes, rows).amax(dim=1)
            self.cache = tile_max if self.cache is None else torch.maximum(self.cache, tile_max)
        else:
            if kind == InputRangeCalibrationType.MOVING_STD:
                alpha = mod.rpu_config.pre_post.input_range.init_std_alpha
                val = alpha * F.sliced_std(mod.in_sizes, rows)
            elif self.quantile == 1.0:
                val = F.sliced_abs_max(mod.in_sizes, rows).amax(dim=1).float()
            else:
                val = torch.stack([rows[:, lo:hi].float().flatten().quantile(self.quantile)
                                   for _, lo, hi in _tile_slices(mod.in_sizes)])
            # running mean over the batches seen so far, in fp32 like the reference's mixed
            # Python-float / int32-tensor expression (`calibration.py:136-139`)
            idx = mod.input_range_update_idx.data.float()
            new = (mod.input_range.data.float() * idx + val.float()) / (idx + 1.0)
            mod.input_range.data.copy_(new.to(mod.input_range.dtype))
            mod.input_range_update_idx.data += 1


@torch.no_grad()
def calibrate_input_ranges(model: Module, calibration_type: InputRangeCalibrationType, dataloader: Iterable,
                           quantile: float = 0.99995, max_samples: int = 1000,
                           std_alpha: Optional[float] = None, verbose: bool = False) -> None:
    """Derive static input ranges for every analog layer of ``model`` from calibration data.

    ``dataloader`` yields ``(args, kwargs)`` pairs that are passed to ``model``.  The layers must
    run without an input range and without a DAC (``inp_res <= 0``), in eval mode; on return
    their ``rpu_config`` has the input range enabled (static) and ``input_range`` holds the
    calibrated values.  Same contract as the reference (`calibration.py:158-320`).
    """
    layers = _named_analog_layers(model)
    if not layers:
        raise ConfigError("The model has no analog layers to calibrate.")
    if calibration_type in (InputRangeCalibrationType.NONE, None):
        raise ConfigError(f"Unknown InputRangeCalibrationType {calibration_type}")
    sample = layers[0][1]
    if sample.rpu_config.pre_post.input_range.enable:
        raise ConfigError("You can only calibrate input ranges for models that don't have input ranges.")
    if sample.rpu_config.forward.inp_res > 0:
        raise ConfigError("When calibrating the input ranges, the input res must be infinite (-1 or 0)")
    if sample.training:
        raise ConfigError("Calibration can only be done in test mode.")
    moving = calibration_type in (InputRangeCalibrationType.MOVING_QUANTILE, InputRangeCalibrationType.MOVING_STD)

    collectors: Dict[str, _Collector] = {}
    restored: Dict[str, object] = {}
    handles = []
    for name, layer in layers:
        n_tiles = len(layer.in_sizes)
        dev, dtype = layer.weight.device, layer.weight.dtype
        if moving:
            # the moving statistics live in the layer's own range parameter, which is active
            # (as a fixed clamp) while the calibration batches run
            irp = layer.rpu_config.pre_post.input_range
            init_value = irp.init_value
            irp.enable, irp.dynamic, irp.learn_input_range, irp.init_value = True, False, True, 3.0
            if std_alpha is not None:
                irp.init_std_alpha = std_alpha
            layer.input_range = Parameter(torch.full((n_tiles,), float(init_value), dtype=dtype, device=dev),
                                          requires_grad=True)
            layer.input_range_update_idx = Parameter(torch.zeros(n_tiles, dtype=dtype, device=dev),
                                                     requires_grad=False)
        # what the layer gets back afterwards: its configuration with the noise sources intact
        restored[name] = deepcopy(layer.rpu_config)
        layer.rpu_config.forward.out_noise = 0.0
        layer.rpu_config.modifier.noise_type = WeightNoiseInjectionType.NONE
        collectors[name] = _Collector(layer, calibration_type, quantile, max_samples)
        handles.append(layer.register_forward_pre_hook(collectors[name], with_kwargs=True))

    batches = dataloader
    if verbose:
        from tqdm import tqdm  # pylint: disable=import-outside-toplevel
        batches = tqdm(dataloader)
    try:
        for args, kwargs in batches:
            model(*args, **kwargs)
    finally:
        for handle in handles:
            handle.remove()

    for name, layer in layers:
        n_tiles = len(layer.in_sizes)
        dev, dtype = layer.weight.device, layer.weight.dtype
        cfg = restored[name]
        layer.input_range_update_idx = Parameter(torch.full((n_tiles,), float("-inf"), dtype=dtype, device=dev),
                                                 requires_grad=False)
        if not moving:
            irp = cfg.pre_post.input_range
            irp.enable = True
            ranges = torch.full((n_tiles,), float(irp.init_value), dtype=dtype, device=dev)
            cache = collectors[name].cache
            if cache is not None:
                if calibration_type == InputRangeCalibrationType.CACHE_QUANTILE:
                    for t, lo, hi in _tile_slices(layer.in_sizes):
                        ranges[t] = cache[:, lo:hi].flatten().quantile(quantile).item()
                else:
                    ranges = cache.to(dtype)
            layer.input_range = Parameter(ranges, requires_grad=irp.learn_input_range)
        layer.rpu_config = cfg
