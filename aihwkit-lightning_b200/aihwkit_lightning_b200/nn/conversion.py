"""Swap torch layers for their analog counterparts and back.

Same arguments, traversal and results as the reference's ``convert_to_analog`` /
``convert_to_digital`` (`nn/conversion.py:71-295`): the module itself is converted when its class
is in the map, then its children -- a child that has children of its own is descended into
(after its own conversion, which is how ``nn.Sequential`` and the recurrent modules are
handled), a leaf is converted through ``from_digital`` -- ``exclude_modules`` holds full dotted
names, every converted layer gets its own deep copy of the config passed through
``specific_rpu_config_fun``, and a root that is not analog itself is wrapped in
``AnalogWrapper`` when ``ensure_analog_root`` is set.
"""
from copy import deepcopy
from typing import Callable, Dict, List, Optional, Set, Type

from ..exceptions import ArgumentError
from torch.nn import GRU, LSTM, RNN, Conv1d, Conv2d, Conv3d, Linear, Module, Sequential

from .modules import (
    AnalogConv1d,
    AnalogConv2d,
    AnalogConv3d,
    AnalogLayerBase,
    AnalogLinear,
    AnalogRNN,
    AnalogSequential,
    AnalogWrapper,
)

_DEFAULT_CONVERSION_MAP: Dict[Type, Type] = {
    Linear: AnalogLinear,
    Conv1d: AnalogConv1d,
    Conv2d: AnalogConv2d,
    Conv3d: AnalogConv3d,
    Sequential: AnalogSequential,
    LSTM: AnalogRNN,
    GRU: AnalogRNN,
    RNN: AnalogRNN,
}
_DEFAULT_DIGITAL_CONVERSION_SET = {*_DEFAULT_CONVERSION_MAP.values()}


def specific_rpu_config_id(module_name: str, module: Module, rpu_config):
    """Default ``specific_rpu_config_fun``: every layer keeps the generic config."""
    # pylint: disable=unused-argument
    return rpu_config


def convert_to_analog(module: Module, rpu_config, conversion_map: Optional[Dict] = None,
                      specific_rpu_config_fun: Optional[Callable] = None, module_name: str = "",
                      ensure_analog_root: bool = True, exclude_modules: Optional[List[str]] = None,
                      inplace: bool = False, verbose: bool = False) -> Module:
    """Return ``module`` with every layer of ``conversion_map`` replaced through ``from_digital``."""
    exclude_modules = exclude_modules or []
    if not inplace:
        module = deepcopy(module)
    if conversion_map is None:
        conversion_map = _DEFAULT_CONVERSION_MAP
    if not isinstance(conversion_map, dict):
        raise ArgumentError("Conversion map should be a dictionary")
    config_fun = specific_rpu_config_fun or specific_rpu_config_id

    def make(mod: Module, name: str) -> Module:
        target = conversion_map[type(mod)]
        if verbose:
            print(f"Converted '{name}' to '{target.__name__}'.")
        return target.from_digital(mod, config_fun(name, mod, deepcopy(rpu_config)))

    converted = module
    if type(module) in conversion_map and module_name not in exclude_modules:
        converted = make(module, module_name)
        if inplace:
            conversion_map[type(module)].move_to_meta(module)  # frees the digital copy at once

    replacements = {}
    for name, child in converted.named_children():
        full_name = f"{module_name}.{name}" if module_name else name
        if full_name in exclude_modules:
            continue
        if next(child.named_children(), None) is not None:
            replacements[name] = convert_to_analog(child, rpu_config, conversion_map, config_fun, full_name, True,
                                                   exclude_modules, True, verbose)
        elif type(child) in conversion_map:
            replacements[name] = make(child, full_name)
    for name, new_child in replacements.items():
        converted._modules[name] = new_child  # pylint: disable=protected-access

    if ensure_analog_root and not module_name and not isinstance(converted, AnalogLayerBase):
        return AnalogWrapper(converted)
    return converted


def convert_to_digital(module: Module, conversion_set: Optional[Set] = None, module_name: str = "",
                       inplace: bool = False) -> Module:
    """Inverse of :func:`convert_to_analog`: every analog layer of ``conversion_set`` (and any
    ``AnalogWrapper``) becomes its torch counterpart through ``to_digital``."""
    if not inplace:
        module = deepcopy(module)
    if conversion_set is None:
        conversion_set = _DEFAULT_DIGITAL_CONVERSION_SET
    if not isinstance(conversion_set, set):
        raise ArgumentError("Conversion set should be a set")

    def unmake(mod: Module) -> Module:
        if not hasattr(type(mod), "to_digital"):
            raise ArgumentError(
                None, "The conversion set should only contain analog layers that support `to_digital` conversion.")
        return type(mod).to_digital(mod)

    if type(module) in conversion_set or isinstance(module, AnalogWrapper):
        module = unmake(module)
    replacements = {}
    for name, child in module.named_children():
        full_name = f"{module_name}.{name}" if module_name else name
        if next(child.named_children(), None) is not None:
            replacements[name] = convert_to_digital(child, conversion_set, full_name, inplace=True)
        elif type(child) in conversion_set:
            replacements[name] = unmake(child)
    for name, new_child in replacements.items():
        module._modules[name] = new_child  # pylint: disable=protected-access
    return module


__all__ = ["convert_to_analog", "convert_to_digital", "specific_rpu_config_id", "AnalogLayerBase"]
