"""``AnalogOptimizer``: wraps any torch optimizer and clips the analog weights after each step.

Same construction as the reference (`optim/analog_optimizer.py:23-79`):
``AnalogOptimizer(SGD, model.analog_layers, model.parameters(), lr=0.1)`` returns an instance
of a class that derives from both ``AnalogOptimizer`` and ``SGD``.
"""
from types import new_class
from typing import Any, Callable, Dict, Generator, Type

from torch.optim import Optimizer


class AnalogOptimizer(Optimizer):
    """Generic wrapper: ``step()`` of the wrapped optimizer, then ``clip_weights()`` of every
    analog layer (a fused CUDA std + clamp per layer)."""

    SUBCLASSES: Dict[str, Type] = {}

    def __new__(cls, optimizer_cls: Type, *_: Any, **__: Any) -> "AnalogOptimizer":
        name = f"{cls.__name__}{optimizer_cls.__name__}"
        if name not in cls.SUBCLASSES:
            cls.SUBCLASSES[name] = new_class(name, (cls, optimizer_cls), {})
        return super().__new__(cls.SUBCLASSES[name])

    # pylint: disable=unused-argument
    def __init__(self, _: Type, analog_layers: Callable[[], Generator], *args: Any, **kwargs: Any):
        super().__init__(*args, **kwargs)

        def clip_all(*_a: Any, **_k: Any) -> None:
            for layer in analog_layers():
                layer.clip_weights()

        self.register_step_post_hook(clip_all)
