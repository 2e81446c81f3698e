"""Calibrators with the collect / compute_amax / reset contract of
``modelopt/torch/quantization/calib/``."""
from .calibrator import _Calibrator
from .histogram import HistogramCalibrator, calibrate_weights
from .max import MaxCalibrator

__all__ = ["_Calibrator", "MaxCalibrator", "HistogramCalibrator", "calibrate_weights"]
