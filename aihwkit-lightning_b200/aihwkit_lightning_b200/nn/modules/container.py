"""Analog-aware containers: modules that hold analog layers without being one.

Mirrors the reference's ``nn/modules/container.py:25-111``: ``AnalogSequential`` is an
``nn.Sequential`` with the analog-layer iteration helpers, ``AnalogWrapper`` grafts those helpers
onto an arbitrary module by creating (once per wrapped class) a subclass of both, sharing the
wrapped module's ``__dict__`` -- parameters are shared by reference, state-dict keys do not
change, and ``isinstance(wrapped, OriginalClass)`` keeps holding.
"""
from collections import OrderedDict
from types import new_class
from typing import Any, Dict, Optional, Type

from torch.nn import Module, Sequential

from .base import AnalogLayerBase


class AnalogContainerBase(AnalogLayerBase):
    """Marks a module whose analog work is done by its children."""

    IS_CONTAINER: bool = True


class AnalogSequential(AnalogContainerBase, Sequential):
    """``nn.Sequential`` that knows its analog layers (`container.py:31-56`)."""

    @classmethod
    def from_digital(cls, module: Sequential, *_: Any, **__: Any) -> "AnalogSequential":
        """Re-house the children of ``module`` (by reference, names kept)."""
        return cls(OrderedDict(module.named_children()))

    @classmethod
    def to_digital(cls, module: "AnalogSequential", *_: Any, **__: Any) -> Sequential:
        return Sequential(OrderedDict(module.named_children()))


class AnalogWrapper(AnalogContainerBase):
    """Adds the analog-layer helpers to any module (`container.py:59-111`).

    ``AnalogWrapper(model)`` returns an object of a class derived from both ``AnalogWrapper``
    and ``type(model)``; the original ``model`` must not be used afterwards, its tensors are
    shared.
    """

    SUBCLASSES: Dict[str, Type] = {}

    def __new__(cls, module: Optional[Module] = None, **__: Any) -> "AnalogWrapper":
        if module is None:  # deepcopy / pickle construct without arguments
            return super().__new__(cls)
        wrapped_cls = type(module)
        name = f"{cls.__name__}{wrapped_cls.__name__}"
        # keyed by the class object as well: two unrelated classes may share a name
        key = f"{name}@{id(wrapped_cls)}"
        if key not in cls.SUBCLASSES:
            cls.SUBCLASSES[key] = new_class(name, (cls, wrapped_cls), {})
        return super().__new__(cls.SUBCLASSES[key])

    def __init__(self, module: Module):  # pylint: disable=super-init-not-called
        self.__dict__.update(module.__dict__)

    def __reduce_ex__(self, protocol):
        # the dynamically created subclass is not importable by name: rebuild it from the
        # wrapped class on unpickling / deepcopy
        wrapped_cls = type(self).__bases__[1]
        return (_rebuild_wrapper, (wrapped_cls, self.__dict__))

    @classmethod
    def from_digital(cls, module: Module, *_: Any, **__: Any) -> "AnalogWrapper":
        return cls(module)

    @classmethod
    def to_digital(cls, module: "AnalogWrapper", *_: Any, **__: Any) -> Module:
        """The wrapped class again, sharing the state."""
        digital_cls = type(module).__bases__[1]
        plain = digital_cls.__new__(digital_cls)
        plain.__dict__ = module.__dict__
        return plain

    def quantize_weights(self) -> None:
        """Quantise the weights of every analog layer below, in place."""
        for layer in self.analog_layers():
            layer.quantize_weights()


def _rebuild_wrapper(wrapped_cls: Type, state: dict) -> AnalogWrapper:
    shell = wrapped_cls.__new__(wrapped_cls)
    shell.__dict__ = state
    return AnalogWrapper(shell)


__all__ = ["AnalogContainerBase", "AnalogSequential", "AnalogWrapper"]
