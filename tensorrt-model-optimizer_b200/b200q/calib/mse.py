"""MSE calibrator (reference: modelopt/torch/quantization/calib/mse.py:29-177): tries
``num_steps`` amax candidates ``initial_amax * linspace(start, stop, num_steps)``, accumulates the
squared error between the tensor and its fake-quantised value for each, and returns the candidate
with the smallest error (per tensor, or per channel along ``axis``)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..utils import convert_quantization_axis_to_reduce_axis
from .calibrator import _Calibrator

__all__ = ["MseCalibrator"]


class MseCalibrator(_Calibrator):
    def __init__(self, amax, axis=None, num_steps=10, start_multiplier=0.25, stop_multiplier=4.0,
                 quant_func=None, error_func=None):
        super().__init__(num_bits=None, axis=axis, unsigned=None)
        self._initial_amax = amax
        self._num_steps = num_steps
        self._start_multiplier = start_multiplier
        self._stop_multiplier = stop_multiplier
        self._quant_func = quant_func
        self._error_func = error_func
        self.reset()

    @torch.no_grad()
    def collect(self, x):
        if self._quant_func is None:
            raise RuntimeError("Quantization function not set. Msecalibrator requires a quant_func to be provided.")
        x = x.detach().to(dtype=torch.float32)
        multipliers = torch.linspace(self._start_multiplier, self._stop_multiplier, steps=self._num_steps,
                                     device=x.device)
        red = convert_quantization_axis_to_reduce_axis(x, self._axis)
        for step, m in enumerate(multipliers):
            # candidate = initial * multiplier with the rounding the reference gets on CPU: the
            # product is formed in fp32 and rounded to the amax dtype (a 0-dim amax promotes to fp32).
            # (On CUDA torch would first round the 0-dim multiplier to the amax dtype.)
            a = self._initial_amax
            cand = a.float() * m if a.dim() == 0 else (a.float() * m).to(a.dtype)
            xq = self._quant_func(x, cand)
            err = self._error_func(x, xq) if self._error_func is not None else F.mse_loss(x, xq, reduction="none")
            loss = err.sum() if red is None else err.sum(dim=red)
            if self._candidate_amaxs[step] is None:
                self._candidate_amaxs[step] = cand
            if self._losses_sum[step] is None:
                self._losses_sum[step] = loss.clone()
            else:
                self._losses_sum[step] += loss

    def reset(self):
        self._losses_sum = [None] * self._num_steps
        self._candidate_amaxs = [None] * self._num_steps
        self._amax = None

    @torch.no_grad()
    def compute_amax(self, verbose: bool = False):
        first = next((l for l in self._losses_sum if l is not None), None)
        if first is None:
            return None
        losses = torch.stack([l if l is not None else torch.full_like(first, float("inf")) for l in self._losses_sum])
        best = torch.argmin(losses, dim=0)
        if first.ndim == 0:
            self._amax = self._candidate_amaxs[best.item()]
        else:
            cands = torch.stack([c.reshape(-1) if c is not None else torch.zeros_like(first) for c in self._candidate_amaxs])
            self._amax = cands[best, torch.arange(best.shape[0], device=best.device)].reshape(self._initial_amax.shape)
        return self._amax
