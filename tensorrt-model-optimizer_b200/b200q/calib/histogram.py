"""Histogram calibrator (reference: modelopt/torch/quantization/calib/histogram.py:35-343).

The reference fixes the bin width with the first batch (max / num_bins) and, when a later batch
exceeds the range, extends the number of bins at that width before binning it.  Here the first
batch fixes the width the same way (one abs-max pass), and every batch is binned by ONE kernel
into an open-ended histogram of ``CAPACITY_FACTOR * num_bins`` 64-bit device counters of that
width: a larger later batch simply lands in higher bins, with no range pass and no host round
trip per batch.  How many bins are live (the reference's ``_num_bins``) is read from the counters
when they are needed.  Samples beyond the capacity, NaN and inf are counted apart and make the
read-out raise.  Integer counters make the result independent of batch order and summable across
data-parallel ranks (``b200q.dist.sync_histograms``).

``compute_amax`` offers "percentile", "entropy" and "mse" on the GPU (one CTA per candidate clip point
for the searches the reference runs as host loops), and all three on the host for counters held
in CPU memory.  "mse" follows the algorithm the reference documents (minimise the count-weighted
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
    CAPACITY_FACTOR = 16   # later batches may reach 16x the first batch's maximum

    def __init__(self, num_bits=8, axis=None, unsigned=False, num_bins=2048, grow_method=None,
                 skip_zeros=False, torch_hist=True):
        super().__init__(num_bits, axis, unsigned)
        if axis is not None:
            raise NotImplementedError("Calibrator histogram collection only supports per tensor scaling")
        self._skip_zeros = skip_zeros
        self._init_bins = num_bins     # bins of the first batch's range
        self._num_bins = num_bins      # live bins (grows; refreshed by _resolve)
        self._calib_hist = None        # int64 [capacity] on the device; first _num_bins are live
        self._calib_bin_edges = None   # fp32 [_num_bins + 1] on the device
        self._range0 = None            # python float: right edge of bin _init_bins - 1
        self._overflow = None          # int64 [1] on the device
        self._stale = False            # counters changed since _num_bins was last read from them

    # ---- range management ------------------------------------------------------------------
    def set_range(self, x_max: float, device):
        """Fix the bin width (x_max / num_bins) before the first batch — also the way all
        data-parallel ranks get the same width."""
        assert self._calib_hist is None, "range already set"
        self._calib_hist = torch.zeros(self._init_bins * self.CAPACITY_FACTOR, dtype=torch.int64, device=device)
        self._overflow = torch.zeros(1, dtype=torch.int64, device=device)
        self._calib_bin_edges = torch.linspace(0, x_max, self._init_bins + 1, device=device)
        self._range0 = float(self._calib_bin_edges[-1])
        self._num_bins = self._init_bins

    @property
    def _width(self):
        return None if self._calib_bin_edges is None else float(self._calib_bin_edges[1] - self._calib_bin_edges[0])

    def _resolve(self):
        """Bring ``_num_bins`` / ``_calib_bin_edges`` up to date with the device counters."""
        if not self._stale:
            return
        self._stale = False
        # one device->host copy: the overflow count and the number of live bins past _num_bins
        tail = self._calib_hist[self._num_bins:]
        if tail.numel():
            live = ((tail != 0) * torch.arange(1, tail.numel() + 1, device=tail.device)).max()
        else:
            live = torch.zeros((), dtype=torch.int64, device=self._calib_hist.device)
        overflow, live = torch.stack([self._overflow[0], live]).tolist()
        if overflow > 0:
            raise RuntimeError(
                f"HistogramCalibrator: {overflow} samples were NaN, inf or beyond "
                f"{self.CAPACITY_FACTOR}x the range of the first batch ({self._range0}); they were not binned.")
        if live:
            n = self._num_bins + live
            width = self._calib_bin_edges[1] - self._calib_bin_edges[0]
            self._calib_bin_edges = torch.arange(n + 1, device=self._calib_hist.device, dtype=torch.float32) * width
            self._num_bins = n

    def _load_counts(self, counts: torch.Tensor):
        """Replace the live counters (used after a cross-rank sum); bins beyond stay empty."""
        n = counts.numel()
        if n > self._num_bins:
            width = self._calib_bin_edges[1] - self._calib_bin_edges[0]
            self._calib_bin_edges = torch.arange(n + 1, device=counts.device, dtype=torch.float32) * width
            self._num_bins = n
        if self._calib_hist.numel() < n:
            self._calib_hist = torch.zeros(n, dtype=torch.int64, device=counts.device)
        self._calib_hist.zero_()
        self._calib_hist[:n] = counts
        self._stale = False

    @torch.no_grad()
    def collect(self, x):
        x = x.detach()
        if not x.is_floating_point() or x.dtype == torch.float64:
            x = x.float()
        if self._skip_zeros:   # the reference's option: exact zeros are not samples (a masked copy)
            x = x[x != 0]
            if x.numel() == 0:
                return
        if self._calib_hist is None:
            self.set_range(float(ops.amax_tensor(x)), x.device)
        ops.hist_collect_open(x, self._calib_hist, self._init_bins, self._range0, self._overflow)
        self._stale = True

    def reset(self):
        self._calib_bin_edges = None
        self._calib_hist = None
        self._overflow = None
        self._range0 = None
        self._num_bins = self._init_bins
        self._stale = False

    # ---- read-out -------------------------------------------------------------------------------
    @property
    def hist(self):
        if self._calib_hist is None:
            return None
        self._resolve()
        return self._calib_hist[: self._num_bins]

    def compute_amax(self, method: str, *, stride: int = 1, start_bin: int = 128, percentile: float = 99.99):
        if self._calib_hist is None:
            return None
        self._resolve()
        if method == "percentile":
            if percentile < 0 or percentile > 100:
                raise ValueError("Invalid percentile. Must be in range 0 <= percentile <= 100.")
            return ops.hist_percentile(self._calib_hist, self._num_bins, self._calib_bin_edges, 0.0, percentile)
        if method == "entropy" and self._calib_hist.is_cuda:
            if isinstance(self._num_bits, tuple):
                raise TypeError("entropy calibration needs an integer num_bits")
            levels = 1 << (self._num_bits - 1 + int(self._unsigned))
            return ops.hist_entropy(self._calib_hist, self._num_bins, self._calib_bin_edges, levels,
                                    start_bin, stride)[0]
        if method == "mse" and self._calib_hist.is_cuda:
            if isinstance(self._num_bits, tuple):
                raise TypeError("mse calibration from a histogram needs an integer num_bits")
            bound = 2.0 ** (self._num_bits - 1 + int(self._unsigned)) - 1
            return ops.hist_mse(self._calib_hist, self._num_bins, self._calib_bin_edges, bound, start_bin, stride)[0]
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
