"""Swap ``nn.Linear`` / ``nn.Conv1d`` / ``nn.Conv2d`` / ``nn.Conv3d`` for their analog counterparts and back.

Covers what the benchmark models need of the reference's ``convert_to_analog`` /
``convert_to_digital`` (`nn/conversion.py:71-295`): same arguments for the Linear/ConvNd
entries of the conversion map, recursion over children, ``exclude_modules`` by name suffix.
"""
from copy import deepcopy
from typing import Dict, List, Optional, Type

from torch.nn import Conv1d, Conv2d, Conv3d, Linear, Module

from .modules import AnalogConv1d, AnalogConv2d, AnalogConv3d, AnalogLayerBase, AnalogLinear

_DEFAULT_CONVERSION_MAP: Dict[Type, Type] = {Linear: AnalogLinear, Conv1d: AnalogConv1d, Conv2d: AnalogConv2d,
                                             Conv3d: AnalogConv3d}
_DEFAULT_DIGITAL_CONVERSION_SET = {AnalogLinear, AnalogConv1d, AnalogConv2d, AnalogConv3d}


def convert_to_analog(module: Module, rpu_config, conversion_map: Optional[Dict] = None,
                      specific_rpu_config_fun=None, module_name: str = "", ensure_analog_root: bool = True,
                      exclude_modules: Optional[List[str]] = None, inplace: bool = False,
                      verbose: bool = False) -> Module:
    """Return ``module`` with every convertible layer replaced through ``from_digital``."""
    del ensure_analog_root
    if not inplace:
        module = deepcopy(module)
    conversion_map = conversion_map or _DEFAULT_CONVERSION_MAP
    exclude_modules = exclude_modules or []

    def excluded(name: str) -> bool:
        return any(name == pat or name.endswith("." + pat) or name.endswith(pat) for pat in exclude_modules)

    def convert(mod: Module, name: str) -> Module:
        if type(mod) in conversion_map and not excluded(name):  # pylint: disable=unidiomatic-typecheck
            cfg = rpu_config
            if specific_rpu_config_fun is not None:
                cfg = specific_rpu_config_fun(name, mod, rpu_config)
            if verbose:
                print(f"converted {name or '<root>'} to {conversion_map[type(mod)].__name__}")
            return conversion_map[type(mod)].from_digital(mod, deepcopy(cfg))
        for child_name, child in list(mod.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            new_child = convert(child, full)
            if new_child is not child:
                setattr(mod, child_name, new_child)
        return mod

    return convert(module, module_name)


def convert_to_digital(module: Module, conversion_set=None, module_name: str = "",
                       inplace: bool = False) -> Module:
    """Inverse of :func:`convert_to_analog`."""
    if not inplace:
        module = deepcopy(module)
    conversion_set = conversion_set or _DEFAULT_DIGITAL_CONVERSION_SET

    def convert(mod: Module) -> Module:
        if type(mod) in conversion_set:  # pylint: disable=unidiomatic-typecheck
            return type(mod).to_digital(mod)
        for child_name, child in list(mod.named_children()):
            new_child = convert(child)
            if new_child is not child:
                setattr(mod, child_name, new_child)
        return mod

    del module_name
    return convert(module)


__all__ = ["convert_to_analog", "convert_to_digital", "AnalogLayerBase"]
