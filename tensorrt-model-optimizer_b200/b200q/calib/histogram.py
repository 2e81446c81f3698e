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

__all__ = ["HistogramCalibrator", "HistogramArena", "attach_histogram_arena", "calibrate_weights"]


class HistogramArena:
    """One allocation for the counters of many histogram calibrators.

    ``counts`` is int64 ``[Q, capacity]``, ``overflow`` int64 ``[Q]`` and ``ranges`` fp32 ``[Q]`` (the first
    batch's abs-max of each calibrator = right edge of its bin ``num_bins - 1``); calibrator ``i`` works on
    row ``i`` of each.  What this buys:

    * the first batch fixes a calibrator's range on the DEVICE (the abs-max kernel writes its slot, the
      binning kernel reads it): no host round trip per calibrator;
    * the data-parallel exchange is in place: one broadcast of ``ranges``, one SUM all-reduce of ``counts``
      (``b200q.dist``), no packing or unpacking;
    * the live length of every histogram is read back with one copy (``resolve``);
    * calibrators that are handed the very same tensor one after the other (the q/k/v or gate/up input
      quantisers of a layer) share one binning pass: a collect is held back until the next collect shows
      whether it is for the same tensor, and up to four calibrators are served by one launch.  Two
      calibrators can share only if they have shared every batch since their first (they then alias one
      range slot); the held-back tensor is kept alive, and a tensor that was modified in place before its
      pass ran raises.
    """

    MAX_SHARE = 4

    def __init__(self, calibrators):
        self.cals = list(calibrators)
        if not self.cals:
            raise ValueError("no calibrators")
        self.num_bins = self.cals[0]._init_bins
        self.capacity = self.num_bins * HistogramCalibrator.CAPACITY_FACTOR
        for i, c in enumerate(self.cals):
            if c._init_bins != self.num_bins or c._calib_hist is not None or c._arena is not None:
                raise ValueError("an arena takes fresh calibrators of one bin count")
            c._arena, c._arena_index = self, i
        self.counts = self.overflow = self.ranges = None
        self._last_range = None   # (key, calibrator, tensor) of the latest first-batch observation
        self._pending = None      # (key, tensor, [calibrators]) of the collect that is held back
        self._stale = False
        self.observe_only = False  # collect() fixes ranges and bins nothing (the pass before a range broadcast)

    def _allocate(self, device):
        q = len(self.cals)
        self.counts = torch.zeros((q, self.capacity), dtype=torch.int64, device=device)
        self.overflow = torch.zeros(q, dtype=torch.int64, device=device)
        self.ranges = torch.zeros(q, dtype=torch.float32, device=device)
        for i, c in enumerate(self.cals):
            c._calib_hist = self.counts[i]
            c._overflow = self.overflow[i:i + 1]
            c._range_dev = self.ranges[i:i + 1]

    @staticmethod
    def _key(x):
        return (x.data_ptr(), x._version, tuple(x.shape), tuple(x.stride()), x.dtype, x.device)

    def observe_range(self, cal, x):
        """First batch of ``cal``: its abs-max becomes the range.  A calibrator whose first batch is the
        tensor another calibrator has just observed aliases that calibrator's slot instead of reading
        the tensor again."""
        if self.counts is None:
            self._allocate(x.device)
        key = self._key(x)
        last = getattr(self, "_last_range", None)
        if last is not None and last[0] == key and last[1]._range_dev is not None:
            cal._range_dev = last[1]._range_dev
        else:
            ops.amax_tensor(x, out=cal._range_dev)
            self._last_range = (key, cal, x)
        cal._ranged = True

    def submit(self, cal, x):
        key = self._key(x)
        p = self._pending
        if (p is not None and p[0] == key and len(p[2]) < self.MAX_SHARE
                and p[2][0]._range_dev.data_ptr() == cal._range_dev.data_ptr() and cal not in p[2]):
            p[2].append(cal)
            return
        self.flush()
        last = getattr(self, "_last_range", None)
        if last is not None and last[0] != key:
            self._last_range = None
        self._pending = (key, x, [cal])

    def flush(self):
        p, self._pending = self._pending, None
        if p is None:
            return
        key, x, cals = p
        if x._version != key[1]:
            raise RuntimeError("HistogramArena: a tensor was modified in place between collect() and the binning "
                               "pass that was held back for it (set HistogramArena.MAX_SHARE = 1 to bin at once)")
        ops.hist_collect_shared(x, [c._calib_hist for c in cals], [c._overflow for c in cals], self.num_bins,
                                cals[0]._range_dev)
        self._stale = True

    def resolve(self):
        """Bring every calibrator's live length, range and bin edges up to date with ONE device->host copy."""
        self.flush()
        self._last_range = None
        if self.counts is None or not self._stale:
            return
        self._stale = False
        idx = torch.arange(1, self.capacity + 1, device=self.counts.device)
        live = ((self.counts != 0) * idx).amax(dim=1)
        # every calibrator's range slot (its own, or the slot of the calibrator whose first batch it shared)
        base = self.ranges.data_ptr()
        slots = torch.tensor([(c._range_dev.data_ptr() - base) // 4 for c in self.cals], device=self.counts.device)
        ranges = self.ranges[slots]
        host = torch.stack([live.double(), self.overflow.double(), ranges.double()]).tolist()
        fresh, grown = [], []
        for c, n_live, over, rng in zip(self.cals, *host):
            if not c._ranged:
                continue
            if over > 0:
                raise RuntimeError(
                    f"HistogramCalibrator: {int(over)} samples were NaN, inf or beyond "
                    f"{HistogramCalibrator.CAPACITY_FACTOR}x the range of the first batch ({rng}); they were not binned.")
            if c._calib_bin_edges is None or c._range0 != rng:
                fresh.append((c, rng))
            n = max(int(n_live), c._init_bins)
            if n > (c._init_bins if fresh and fresh[-1][0] is c else c._num_bins):
                grown.append((c, n, rng))
        # the bin edges of all calibrators by two batched computations instead of one or two launches each
        dev = self.counts.device
        if fresh:
            rows = _batched_linspace(torch.tensor([r for _, r in fresh], dtype=torch.float32, device=dev), self.num_bins + 1)
            for (c, rng), row in zip(fresh, rows):
                c._calib_bin_edges, c._range0, c._num_bins = row, rng, c._init_bins
        if grown:
            width = (torch.tensor([r for _, _, r in grown], dtype=torch.float32, device=dev)
                     / torch.full((), self.num_bins, dtype=torch.float32, device=dev))
            idx = torch.arange(max(n for _, n, _ in grown) + 1, dtype=torch.float32, device=dev)
            rows = idx[None, :] * width[:, None]
            for (c, n, _), row in zip(grown, rows):
                c._calib_bin_edges, c._num_bins = row[:n + 1], n


def _batched_linspace(ends: torch.Tensor, steps: int) -> torch.Tensor:
    """Row i = ``torch.linspace(0, ends[i], steps)`` to the bit, for fp32 ``ends`` on a CUDA device: torch's
    kernel forms the first half as ``step * i`` and the second half as ``end - step * (steps - 1 - i)`` in ONE
    fused multiply-add (a single rounding); the float64 detour below rounds once as well (the product is
    exact in float64).  Checked against torch.linspace in tests/test_calib_arena_gpu.py."""
    step = ends / torch.full((), steps - 1, dtype=torch.float32, device=ends.device)
    idx = torch.arange(steps, dtype=torch.float32, device=ends.device)
    lo = step[:, None] * idx[None, :]
    hi = (ends.double()[:, None] - step.double()[:, None] * ((steps - 1) - idx).double()[None, :]).float()
    return torch.where(idx[None, :] < (steps // 2), lo, hi)


def attach_histogram_arena(model, share_inputs: bool = True):
    """Give all fresh HistogramCalibrators of ``model`` (grouped by bin count) a common arena.  Returns the
    arenas (possibly none)."""
    from ..nn import TensorQuantizer

    groups = {}
    for _, m in model.named_modules():
        if isinstance(m, TensorQuantizer):
            c = getattr(m, "_calibrator", None)
            if isinstance(c, HistogramCalibrator) and c._calib_hist is None and c._arena is None and not c._skip_zeros:
                groups.setdefault(c._init_bins, []).append(c)
    arenas = [HistogramArena(cs) for cs in groups.values()]
    for a in arenas:
        a.MAX_SHARE = HistogramArena.MAX_SHARE if share_inputs else 1
    return arenas


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
        self._arena = None             # HistogramArena this calibrator's counters live in, if any
        self._arena_index = -1
        self._range_dev = None         # fp32 [1] on the device: the range, when it is kept there (arena)
        self._ranged = False

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

    def _set_live(self, n_live: int, range0: float):
        """Arena read-back: live bins and the range the device holds."""
        if self._calib_bin_edges is None or self._range0 != range0:
            self._calib_bin_edges = torch.linspace(0, range0, self._init_bins + 1, device=self._calib_hist.device)
            self._range0 = range0
            self._num_bins = self._init_bins
        n = max(n_live, self._init_bins)
        if n > self._num_bins:
            width = self._calib_bin_edges[1] - self._calib_bin_edges[0]
            self._calib_bin_edges = torch.arange(n + 1, device=self._calib_hist.device, dtype=torch.float32) * width
            self._num_bins = n

    def observe_range(self, x):
        """Fix the range from ``x`` (the first batch) without binning it."""
        x = x.detach()
        if self._arena is not None:
            self._arena.observe_range(self, x)
        elif self._calib_hist is None:
            self.set_range(float(ops.amax_tensor(x)), x.device)

    def _resolve(self):
        """Bring ``_num_bins`` / ``_calib_bin_edges`` up to date with the device counters."""
        if self._arena is not None:
            self._arena.resolve()
            return
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

    def collect(self, x):   # works on x.detach(): no autograd context needed (it costs microseconds per call)
        x = x.detach()
        if not x.is_floating_point() or x.dtype == torch.float64:
            x = x.float()
        if self._skip_zeros:   # the reference's option: exact zeros are not samples (a masked copy)
            x = x[x != 0]
            if x.numel() == 0:
                return
        if self._arena is not None:
            if not self._ranged:
                self._arena.observe_range(self, x)
            if not self._arena.observe_only:
                self._arena.submit(self, x)
            return
        if self._calib_hist is None:
            self.set_range(float(ops.amax_tensor(x)), x.device)
        ops.hist_collect_open(x, self._calib_hist, self._init_bins, self._range0, self._overflow)
        self._stale = True

    def reset(self):
        if self._arena is not None:
            self._arena.flush()
            if self._calib_hist is not None:
                self._calib_hist.zero_()
                self._overflow.zero_()
            if self._arena.ranges is not None:
                self._range_dev = self._arena.ranges[self._arena_index:self._arena_index + 1]
            self._ranged = False
            self._calib_bin_edges = None
            self._range0 = None
            self._num_bins = self._init_bins
            self._arena._stale = True
            return
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
        if self._calib_hist is None or (self._arena is not None and not self._ranged):
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
    """Calibrate the weight quantiser of every quantised sub-module from its weight alone, with ``method``
    ("max", "mse" or "percentile") regardless of the calibrator the quantiser carries; per output channel
    (axis 0) when ``perchannel``.  The reference builds one numpy histogram per channel on the host
    (modelopt/torch/quantization/calib/histogram.py:346-433); here every channel gets a device histogram
    (one binning launch each) and, for "percentile", all channels of a weight are read out by one launch.
    Each value equals what a HistogramCalibrator fed that tensor or channel returns."""
    from ..utils import convert_quantization_axis_to_reduce_axis, reduce_amax

    for _, module in model.named_modules():
        wq, w = getattr(module, "weight_quantizer", None), getattr(module, "weight", None)
        if wq is None or w is None:
            continue
        w = w.detach()
        axis = 0 if perchannel else None
        if method == "max":
            amax = reduce_amax(w, axis=convert_quantization_axis_to_reduce_axis(w, axis))
        elif method in ("mse", "percentile"):
            if method == "percentile" and (percentile < 0 or percentile > 100):
                raise ValueError("Invalid percentile. Must be in range 0 <= percentile <= 100.")
            parts = [w] if axis is None else [w.select(axis, i) for i in range(w.shape[axis])]
            cals = []
            for part in parts:
                cal = HistogramCalibrator(wq.num_bits, None, wq.unsigned, num_bins=num_bins)
                cal.collect(part.contiguous())
                cals.append(cal)
            if method == "percentile" and w.is_cuda:
                for cal in cals:
                    cal._resolve()
                values = ops.hist_percentile_batch([(c._calib_hist, c._num_bins, c._calib_bin_edges) for c in cals],
                                                   percentile)
            else:
                values = torch.stack([c.compute_amax(method).reshape(()).to(w.device) for c in cals])
            if axis is None:
                amax = values.reshape(())
            else:
                shape = [1] * w.dim()
                shape[axis] = w.shape[axis]
                amax = values.reshape(shape)
        else:
            raise TypeError(f"Unsupported calibration method {method}")
        if amax.numel() == 1:
            amax = amax.reshape(())
        wq.amax = amax.to(w.dtype) if method == "max" else amax
