"""Max calibrator (reference: modelopt/torch/quantization/calib/max.py:26-110).

The running amax lives in one fp32 device buffer that the reduction kernel folds new batches into
with an atomic max, so ``collect`` is a single kernel launch with no host synchronisation.  The
reference's three per-call assertions (non-negative, no inf, no NaN — each a device sync) are made
once, in ``compute_amax``; NaN and inf survive the running max, so nothing is missed.
"""
from __future__ import annotations

import torch

from .. import ops
from ..utils import convert_quantization_axis_to_reduce_axis
from .calibrator import _Calibrator

__all__ = ["MaxCalibrator"]


class MaxCalibrator(_Calibrator):
    def __init__(self, num_bits=8, axis=None, unsigned=False, track_amax=False):
        super().__init__(num_bits, axis, unsigned)
        self._track_amax = track_amax
        if track_amax:
            self._amaxs = []
        self._acc = None        # fp32 running max, flat
        self._shape = None      # keepdims shape of the amax
        self._dtype = None

    @property
    def amaxs(self):
        return self._amaxs

    @staticmethod
    def _plan(x, axis):
        """(outer, n_axis, inner, keepdims shape, permutation or None) of the reduction."""
        red = convert_quantization_axis_to_reduce_axis(x, axis)
        nd = x.dim()
        if red is None or len(red) == nd:
            return None
        keep = [d for d in range(nd) if d not in red]
        shape = [x.shape[d] if d in keep else 1 for d in range(nd)]
        n_axis = 1
        for d in keep:
            n_axis *= x.shape[d]
        if keep == list(range(keep[0], keep[-1] + 1)):
            outer = 1
            for d in range(keep[0]):
                outer *= x.shape[d]
            inner = 1
            for d in range(keep[-1] + 1, nd):
                inner *= x.shape[d]
            return outer, n_axis, inner, shape, None
        inner = 1
        for d in red:
            inner *= x.shape[d]
        return 1, n_axis, inner, shape, [*keep, *red]

    def collect(self, x):   # works on x.detach(): no autograd context needed (it costs microseconds per call)
        x = x.detach()
        plan = self._plan(x, self._axis)
        shape = [] if plan is None else plan[3]
        if x.device.type == "meta":
            self._shape = shape
            return
        n = 1 if plan is None else plan[1]
        if self._acc is None:
            self._acc = torch.zeros(n, dtype=torch.float32, device=x.device)
            self._shape, self._dtype = shape, x.dtype
        elif list(shape) != list(self._shape) or self._acc.numel() != n:
            raise RuntimeError("amax shape changed!")
        target = torch.zeros_like(self._acc) if self._track_amax else self._acc
        if plan is None:
            ops.amax_tensor(x, out=target)
        else:
            outer, n_axis, inner, _, perm = plan
            xx = x if perm is None else x.permute(*perm).contiguous()
            ops.amax_axis3(xx, outer, n_axis, inner, out=target)
        if self._track_amax:
            torch.maximum(self._acc, target, out=self._acc)
            self._amaxs.append(target.reshape(shape).cpu().numpy())

    def reset(self):
        self._acc = None
        self._shape = None

    def compute_amax(self, check: bool = True):
        """The abs-max of everything collected, in the dtype of the collected tensors and with
        keepdims shape (0-dim for per-tensor), or ``None`` if nothing was collected.  ``check=False``
        leaves the nan/inf/negative test (one device->host read) to a caller that tests many values at
        once (``model_calib.load_calib_amax_all``)."""
        if self._acc is None:
            return None
        amax = self._acc.reshape(self._shape).to(self._dtype)
        if check:
            bad = torch.isnan(self._acc).any() | torch.isinf(self._acc).any() | (self._acc < 0).any()
            assert not bool(bad), "detected nan/inf/negative values in amax: check the calibrated tensors"
        return amax

    def __str__(self):
        return f"MaxCalibrator(track_amax={self._track_amax})"

    def __repr__(self):
        return f"MaxCalibrator({super().__repr__()} calib_amax={self._acc} track_amax={self._track_amax})"
