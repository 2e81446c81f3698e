"""Histogram calibrator (reference: modelopt/torch/quantization/calib/histogram.py:35-343).

``collect`` keeps the reference's range rules — the first batch fixes the bin width
(max / num_bins), later batches that exceed the range extend the number of bins at that width —
but runs as two single-pass kernels (abs-max, then binning of |x| into 64-bit device counters)
instead of the abs / float / max / histc chain.  Integer counters make the result independent of
batch order and summable across data-parallel ranks (``b200q.dist.sync_histograms``).

``compute_amax`` offers "percentile" (on the GPU), and "entropy" / "mse" on the host from the
copied counts.  "mse" follows the algorithm the reference documents (minimise the count-weighted
squared error of fake-quantised bin centres); the reference's own implementation passes its
arguments to ``fake_tensor_quant`` in the wrong slots (histogram.py:308) and is not reproduced.
"""
from __future__ import annotations

import math
import warnings

import numpy as np
import torch

from .. import ops
from .calibrator import _Calibrator

__all__ = ["HistogramCalibrator", "calibrate_weights"]


class HistogramCalibrator(_Calibrator):
    def __init__(self, num_bits=8, axis=None, unsigned=False, num_bins=2048, grow_method=None,
                 skip_zeros=False, torch_hist=True):
        super().__init__(num_bits, axis, unsigned)
        if axis is not None:
            raise NotImplementedError("Calibrator histogram collection only supports per tensor scaling")
        if skip_zeros:
            raise NotImplementedError("skip_zeros is not supported by the CUDA histogram")
        self._num_bins = num_bins
        self._calib_hist = None        # int64 [capacity] on the device; first _num_bins are live
        self._calib_bin_edges = None   # fp32 [_num_bins + 1] on the device
        self._width = None             # python float, fixed by the first batch (or by set_range)

    # ---- range management ------------------------------------------------------------------
    def set_range(self, x_max: float, device):
        """Fix the histogram range before the first batch (used to give all data-parallel ranks
        the same bin width)."""
        assert self._calib_hist is None, "range already set"
        self._calib_hist = torch.zeros(self._num_bins, dtype=torch.int64, device=device)
        self._calib_bin_edges = torch.linspace(0, x_max, self._num_bins + 1, device=device)
        self._width = float(self._calib_bin_edges[1] - self._calib_bin_edges[0])

    def _grow(self, x_max_t: torch.Tensor):
        width = self._calib_bin_edges[1] - self._calib_bin_edges[0]
        self._num_bins = int((x_max_t / width).ceil().item())
        self._calib_bin_edges = torch.arange(0, float(x_max_t + width), float(width),
                                             device=self._calib_hist.device, dtype=torch.float32)
        if self._calib_hist.numel() < self._num_bins:
            bigger = torch.zeros(max(self._num_bins, 2 * self._calib_hist.numel()), dtype=torch.int64,
                                 device=self._calib_hist.device)
            bigger[: self._calib_hist.numel()] = self._calib_hist
            self._calib_hist = bigger

    @torch.no_grad()
    def collect(self, x):
        x = x.detach()
        x_max_t = ops.amax_tensor(x)
        if self._calib_hist is None:
            self.set_range(float(x_max_t), x.device)
        elif bool(x_max_t > self._calib_bin_edges[-1]):
            self._grow(x_max_t)
        ops.hist_collect(x, self._calib_hist, self._num_bins, float(self._calib_bin_edges[-1]))

    def reset(self):
        self._calib_bin_edges = None
        self._calib_hist = None

    # ---- read-out -------------------------------------------------------------------------------
    @property
    def hist(self):
        return None if self._calib_hist is None else self._calib_hist[: self._num_bins]

    def compute_amax(self, method: str, *, stride: int = 1, start_bin: int = 128, percentile: float = 99.99):
        if self._calib_hist is None:
            return None
        if method == "percentile":
            if percentile < 0 or percentile > 100:
                raise ValueError("Invalid percentile. Must be in range 0 <= percentile <= 100.")
            return ops.hist_percentile(self._calib_hist, self._num_bins, self._calib_bin_edges, 0.0, percentile)
        counts = self.hist.cpu().numpy()
        edges = self._calib_bin_edges.cpu().numpy()
        if method == "entropy":
            return torch.tensor(float(_entropy_amax(counts, edges, self._num_bits, self._unsigned, stride, start_bin)))
        if method == "mse":
            return torch.tensor(float(_mse_amax(counts, edges, self._num_bits, self._unsigned, stride, start_bin)))
        raise TypeError(f"Unknown calibration method {method}")

    def __str__(self):
        if self._calib_bin_edges is None:
            return "HistogramCalibrator(calib_bin_edges=None)"
        e = self._calib_bin_edges
        return f"HistogramCalibrator(calib_bin_edges=[{e[0]:.3f}, ..., {e[-1]:.3f}]({len(e)}))"

    def __repr__(self):
        return f"HistogramCalibrator({super().__repr__()} calib_bin_edges={self._calib_bin_edges})"


def _entropy_amax(hist, edges, num_bits, unsigned, stride=1, start_bin=128):
    """KL-divergence calibration over candidate clip points (reference histogram.py:210-282):
    for each candidate i the first i bins are merged into 2^(bits-1+unsigned) levels, each level's
    mass is spread evenly over its non-empty bins, and KL(reference || candidate) is taken with the
    clipped tail added to the reference's last bin.  The last minimum wins.  Vectorised per
    candidate with bincount instead of Python loops over bins."""
    if isinstance(num_bits, tuple):
        raise TypeError("entropy calibration needs an integer num_bits")
    bins = np.array(hist, dtype=np.int64)
    bins[0] = bins[1]
    nlev = 1 << (num_bits - 1 + int(unsigned))
    tail = np.concatenate([np.cumsum(bins[::-1])[::-1], [0]])  # tail[i] = sum(bins[i:])
    divs = []
    for i in range(start_bin, len(bins) + 1, stride):
        dig = np.digitize(np.arange(i), np.linspace(0, i, num=nlev + 1)) - 1
        nz = bins[:i] != 0
        mass = np.bincount(dig[nz], weights=bins[:i][nz].astype(np.float64), minlength=nlev)
        cnt = np.bincount(dig[nz], minlength=nlev)
        avg = np.divide(mass, cnt, out=np.zeros(nlev), where=cnt > 0)
        cand = np.where(nz, avg[dig], 0.0)
        ref = bins[:i].astype(np.float64)
        ref[-1] += tail[i]
        p, q = ref / ref.sum(), cand / cand.sum()
        with np.errstate(divide="ignore", invalid="ignore"):
            t = np.where(p > 0, p * np.log(p / q), 0.0)
        t = np.where((p > 0) & (q == 0), np.inf, t)
        divs.append(t.sum())
    divs = np.array(divs)
    last_argmin = len(divs) - 1 - int(np.argmin(divs[::-1]))
    return edges[last_argmin * stride + start_bin]


def _mse_amax(hist, edges, num_bits, unsigned, stride=1, start_bin=128):
    """Clip point minimising the count-weighted squared error of fake-quantised bin centres."""
    counts = np.asarray(hist, dtype=np.float64)
    edges = np.asarray(edges, dtype=np.float64)
    centers = (edges[1:] + edges[:-1]) / 2
    best, best_i = math.inf, start_bin
    if isinstance(num_bits, tuple):
        raise TypeError("mse calibration from a histogram needs an integer num_bits")
    bound = 2.0 ** (num_bits - 1 + int(unsigned)) - 1
    for i in range(start_bin, len(centers), stride):
        amax = centers[i]
        scale = bound / amax
        q = np.clip(np.rint(centers * scale), -bound, bound) / scale
        mse = ((q - centers) ** 2 * counts).mean()
        if mse < best:
            best, best_i = mse, i
    return centers[best_i]


def calibrate_weights(model, method="percentile", perchannel=True, percentile=99.99, num_bins=2048):
    """Not part of the accelerated path: weights are calibrated by ``max_calibrate``."""
    warnings.warn("calibrate_weights is not provided; use b200q.calibrate(model, 'max')")
