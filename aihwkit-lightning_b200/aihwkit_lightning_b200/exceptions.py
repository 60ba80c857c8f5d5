"""Exception types raised at the analog-layer boundary.

Same names and hierarchy as the reference (`src/aihwkit_lightning/exceptions.py:16-33`) so that
``except ConfigError`` written against the reference keeps working; ``KernelError`` is new and
carries a non-zero status of the CUDA library.
"""


class AihwkitException(Exception):
    """Root of all errors raised by this package."""


class ModuleError(AihwkitException):
    """An analog module was built or used wrongly."""


class ArgumentError(AihwkitException):
    """A call received an argument it cannot work with."""


class ConfigError(AihwkitException):
    """The RPU configuration asks for something that is not supported."""


class TorchTileConfigError(ConfigError):
    """Configuration error specific to the tile emulation."""


class KernelError(AihwkitException):
    """The CUDA library returned a non-zero status (bad shape, CUDA error, device-side wait
    that gave up)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"analog_b200 status {status}: {message}")
        self.status = status
