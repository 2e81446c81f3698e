"""Calibrators with the collect / compute_amax / reset contract of
``modelopt/torch/quantization/calib/``."""
from .bias import BiasCalibrator
from .calibrator import _Calibrator
from .histogram import HistogramArena, HistogramCalibrator, attach_histogram_arena, calibrate_weights
from .max import MaxCalibrator
from .mse import MseCalibrator

__all__ = ["_Calibrator", "BiasCalibrator", "MaxCalibrator", "MseCalibrator", "HistogramCalibrator", "HistogramArena",
           "attach_histogram_arena", "calibrate_weights"]
