"""B200-native implementation of the analog linear path of AIHWKIT-Lightning.

Public surface (same names as the reference package):

* ``aihwkit_lightning_b200.nn``        ``AnalogLinear``, ``AnalogConv1d/2d/3d``, ``AnalogRNN`` and its cells,
                                       ``AnalogSequential``, ``AnalogWrapper``, ``convert_to_analog`` / ``convert_to_digital``
* ``aihwkit_lightning_b200.simulator`` ``TorchInferenceRPUConfig`` and its parameter classes / enums
* ``aihwkit_lightning_b200.optim``     ``AnalogOptimizer``
* ``aihwkit_lightning_b200.inference`` ``calibrate_input_ranges``, ``InputRangeCalibrationType``

All arithmetic runs in ``lib/libanalog_b200.so`` (hand-written sm_100a CUDA behind a C ABI);
CPU tensors are rejected, there is no fallback path.
"""
__version__ = "0.1.0"

from . import exceptions, simulator  # noqa: F401
from . import nn, optim  # noqa: F401
from . import inference  # noqa: F401
