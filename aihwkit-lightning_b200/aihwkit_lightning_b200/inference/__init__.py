"""Post-training inference tools."""
from .calibration import InputRangeCalibrationType, calibrate_input_ranges

__all__ = ["InputRangeCalibrationType", "calibrate_input_ranges"]
