"""MSE calibrator (reference: modelopt/torch/quantization/calib/mse.py:29-177): ``num_steps`` candidate
amax values ``initial_amax * linspace(start, stop, num_steps)``; the squared error between a tensor and
its fake-quantised value is accumulated per candidate (per tensor, or per channel along ``axis``) over
all collected batches, and the candidate with the smallest error wins.

Where the quantiser is a plain integer or E4M3 fake quantiser (``fused`` describes it) one kernel launch
evaluates every candidate in a single pass over the batch (``ops.mse_candidates``); any other quantiser,
or a custom ``error_func``, is evaluated candidate by candidate through ``quant_func`` as the reference
does."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops
from ..utils import convert_quantization_axis_to_reduce_axis
from .calibrator import _Calibrator

__all__ = ["MseCalibrator"]


class MseCalibrator(_Calibrator):
    def __init__(self, amax, axis=None, num_steps=10, start_multiplier=0.25, stop_multiplier=4.0,
                 quant_func=None, error_func=None, fused: dict | None = None):
        """``fused``: {"num_bits": int | (4, 3), "unsigned": bool, "narrow_range": bool} when ``quant_func``
        is exactly that fake quantiser applied with the candidate amax (set by ``mse_calibrate``)."""
        super().__init__(num_bits=None, axis=axis, unsigned=None)
        self._initial_amax = amax
        self._num_steps = num_steps
        self._start_multiplier = start_multiplier
        self._stop_multiplier = stop_multiplier
        self._quant_func = quant_func
        self._error_func = error_func
        self._fused = fused
        self.reset()

    def _candidates(self, device):
        """[num_steps] candidate amax tensors of the initial amax's shape.  candidate = initial * multiplier
        with the rounding the reference gets on the CPU: the product is formed in fp32 and rounded to the
        amax dtype (a 0-dim amax promotes to fp32).  (On CUDA torch would first round the 0-dim multiplier
        to the amax dtype.)"""
        mult = torch.linspace(self._start_multiplier, self._stop_multiplier, steps=self._num_steps, device=device)
        a = self._initial_amax.to(device)
        out = []
        for m in mult:
            out.append(a.float() * m if a.dim() == 0 else (a.float() * m).to(a.dtype))
        return out

    def _fused_axis(self, x):
        """Channel axis for the kernel, or False when this collect has to take the candidate loop."""
        if self._fused is None or self._error_func is not None or not x.is_cuda or self._num_steps > 16:
            return False
        axis = self._axis
        if isinstance(axis, (list, tuple)):
            if len(axis) != 1:
                return False
            axis = axis[0]
        if axis is not None and self._initial_amax.numel() != x.shape[axis]:
            return False
        if axis is None and self._initial_amax.numel() != 1:
            return False
        return axis if ops.mse_candidates_supported(x, axis) else False

    @torch.no_grad()
    def collect(self, x):
        if self._quant_func is None:
            raise RuntimeError("Quantization function not set. Msecalibrator requires a quant_func to be provided.")
        x = x.detach()
        cands = self._candidates(x.device)
        for step, c in enumerate(cands):
            if self._candidate_amaxs[step] is None:
                self._candidate_amaxs[step] = c
        axis = self._fused_axis(x)
        if axis is not False:
            channels = 1 if axis is None else x.shape[axis]
            if self._loss_buf is None:
                self._loss_buf = torch.zeros((self._num_steps, channels), dtype=torch.float64, device=x.device)
                for step in range(self._num_steps):
                    prior = self._losses_sum[step]
                    if prior is not None:       # earlier batches went through the loop
                        self._loss_buf[step] += prior.reshape(-1).double()
                    self._losses_sum[step] = self._loss_buf[step].reshape(()) if axis is None else self._loss_buf[step]
            ops.mse_candidates(x, torch.stack([c.float().reshape(-1) for c in cands]), self._loss_buf, axis,
                               self._fused["num_bits"], self._fused["unsigned"], self._fused["narrow_range"])
            return
        x = x.to(dtype=torch.float32)
        red = convert_quantization_axis_to_reduce_axis(x, self._axis)
        for step, c in enumerate(cands):
            xq = self._quant_func(x, c)
            err = self._error_func(x, xq) if self._error_func is not None else F.mse_loss(x, xq, reduction="none")
            loss = err.sum() if red is None else err.sum(dim=red)
            if self._losses_sum[step] is None:
                self._losses_sum[step] = loss.clone()
            else:
                self._losses_sum[step] += loss

    def reset(self):
        self._losses_sum = [None] * self._num_steps
        self._candidate_amaxs = [None] * self._num_steps
        self._loss_buf = None
        self._amax = None

    @torch.no_grad()
    def compute_amax(self, verbose: bool = False):
        have = [l for l in self._losses_sum if l is not None]
        if not have:
            return None
        first = have[0]
        losses = torch.stack([l if l is not None else torch.full_like(first, float("inf")) for l in self._losses_sum])
        best = torch.argmin(losses, dim=0)
        if first.ndim == 0:
            self._amax = self._candidate_amaxs[best.item()]
        else:
            cands = torch.stack([c.reshape(-1) if c is not None else torch.zeros_like(first) for c in self._candidate_amaxs])
            self._amax = cands[best, torch.arange(best.shape[0], device=best.device)].reshape(self._initial_amax.shape)
        return self._amax
