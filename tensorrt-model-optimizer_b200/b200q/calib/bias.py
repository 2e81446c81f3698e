"""Bias calibrator for affine quantisation (reference: modelopt/torch/quantization/calib/bias.py:26-172):
tracks the offset that is subtracted before and added back after quantisation, e.g. per head and
channel for KV-cache tensors.  ``axis`` names the dimensions that are REDUCED (negative or
non-negative); the others keep their extent.  Small reductions on tensors that the calibration
forward has just produced: plain torch reductions on the tensor's device."""
from __future__ import annotations

import torch

from .calibrator import _Calibrator

__all__ = ["BiasCalibrator", "compute_bias", "compute_maxmin", "subtract_bias", "add_bias"]


def _reduce_dims(x: torch.Tensor, axis):
    return tuple(i for i in range(x.dim()) if i in axis or (i - x.dim()) in axis)


def compute_maxmin(inputs: torch.Tensor, axis):
    if axis is None:
        return torch.max(inputs), torch.min(inputs)
    dims = _reduce_dims(inputs, axis)
    return torch.amax(inputs, dim=dims, keepdim=True), torch.amin(inputs, dim=dims, keepdim=True)


def compute_bias(inputs: torch.Tensor, axis, method: str = "mean") -> torch.Tensor:
    """``mean``: the mean over the reduced dimensions; otherwise the mid-range (max + min) / 2."""
    if method == "mean":
        if axis is None:
            return torch.mean(inputs)
        return torch.mean(inputs, dim=_reduce_dims(inputs, axis), keepdim=True)
    hi, lo = compute_maxmin(inputs, axis)
    return (hi + lo) / 2


def subtract_bias(inputs: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    return inputs - bias


def add_bias(inputs: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    return (inputs + bias).view(inputs.shape)


class BiasCalibrator(_Calibrator):
    def __init__(self, method: str = "mean", axis=None):
        super().__init__(axis=axis)
        if method not in ("mean", "max_min"):
            raise ValueError(f"Unsupported method: {method}")
        self._method = method
        self.reset()

    def collect(self, x: torch.Tensor):
        if self._method == "mean":   # running average over the batches seen so far
            b = compute_bias(x, self._axis, "mean")
            self._calib_bias = b if self._calib_bias is None else (self._calib_bias * self._cnt + b) / (self._cnt + 1)
            self._cnt += 1
        else:                        # running extremes, mid-range of those
            hi, lo = compute_maxmin(x, self._axis)
            self._calib_max = hi if self._calib_max is None else torch.max(self._calib_max, hi)
            self._calib_min = lo if self._calib_min is None else torch.min(self._calib_min, lo)
            self._calib_bias = (self._calib_max + self._calib_min) / 2

    def compute_bias(self):
        return self._calib_bias

    def compute_dynamic_bias(self, inputs):
        return compute_bias(inputs, self._axis, method=self._method)

    def reset(self):
        self._calib_bias = None
        self._calib_max = None
        self._calib_min = None
        self._cnt = 0
